"""Getting a call's rois onto the device without a blocking copy, an allocation or a cast kernel.

The reference builds the rois of every augmentation call as a pageable ``torch.FloatTensor`` and moves it with
``.to(device)`` -- a synchronous copy -- once per field, then casts it on the device to the image's dtype
(medvision/aug_cuda_batch/aug_spatial.py:419-431, medvision/ops/cuda_fun_tools.py:82).  The parameters of a
transform are drawn on the host (numpy's generator; the order of the draws is part of the interface), so one
small upload per call is inherent.  Here it is ONE asynchronous copy from pinned memory into a device buffer that
is kept across calls, carrying the rois in float32 (for label fields) and, rounded on the host exactly as the
device cast rounds, in float16 (for half images): no allocation, no synchronisation, no cast kernel.
"""
import torch

_SLOTS = 4  # calls that may be in flight before a staging slot is reused


class _Stage:
    def __init__(self, device, capacity):
        self.capacity = capacity  # roi values per slot
        per_slot = capacity * 6   # bytes: float32 + float16 copy of every value
        self.host = [torch.empty(per_slot, dtype=torch.uint8, pin_memory=True) for _ in range(_SLOTS)]
        self.dev = [torch.empty(per_slot, dtype=torch.uint8, device=device) for _ in range(_SLOTS)]
        self.free = [None] * _SLOTS  # event recorded after the last kernels that read the slot
        self.next = 0


_stages = {}


def stage_rois(rois, device):
    """rois: CPU float32 (R, K).  Returns (rois_f32, rois_f16, release): device views of the staged rois and a
    function to call once every kernel that reads them has been launched on the current stream."""
    device = torch.device(device)
    n = rois.numel()
    st = _stages.get(device)
    if st is None or st.capacity < n:
        st = _stages[device] = _Stage(device, max(1024, 2 * n))
    k = st.next
    st.next = (k + 1) % _SLOTS
    capturing = torch.cuda.is_current_stream_capturing()
    if st.free[k] is not None and not capturing:
        st.free[k].synchronize()  # the kernels of the call that last used this slot are done (a few calls back)
    host, dev = st.host[k], st.dev[k]
    rois = rois.contiguous()
    host[:4 * n].view(torch.float32).copy_(rois.view(-1))
    host[4 * n:6 * n].view(torch.float16).copy_(rois.view(-1))  # round-to-nearest-even, as the device cast
    with torch.cuda.device(device):
        dev[:6 * n].copy_(host[:6 * n], non_blocking=True)
    f32 = dev[:4 * n].view(torch.float32).view(rois.shape)
    f16 = dev[4 * n:6 * n].view(torch.float16).view(rois.shape)

    def release():
        if not torch.cuda.is_current_stream_capturing():
            ev = st.free[k] or torch.cuda.Event()
            ev.record(torch.cuda.current_stream(device))
            st.free[k] = ev
    return f32, f16, release
