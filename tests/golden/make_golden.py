"""Generate tests/golden/reference_cuda.npz from the reference's OWN CUDA kernels.

Run on a machine with a B200 and a built ``oracle/_ref/mvref_C*.so``:

    python tests/golden/make_golden.py [output.npz]
    python tests/golden/make_golden.py offset          # -> reference_offset_cuda.npz

For every case of ``cases.py`` the seeded inputs go through the reference's forward and
backward kernels; inputs are NOT stored (they are regenerated from the seed), outputs are.
Half tensors are stored as their uint16 bit patterns.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, HERE)

import cases  # noqa: E402
from oracle import ref  # noqa: E402


def to_np(t):
    t = t.detach().cpu().contiguous()
    return t.view(torch.int16).numpy().view(np.uint16) if t.dtype == torch.float16 else t.numpy()


def main_offset():
    """apply_offset_2d/3d through the reference's deform_2d / deform_3d kernels."""
    out_path = os.path.join(HERE, "reference_offset_cuda.npz")
    blobs = {}
    for name, case in cases.offset_cases():
        img, off = cases.make_offset_inputs(case)
        blobs[name] = to_np(ref.apply_offset(img.cuda(), off.cuda(), case["order"]))
    np.savez_compressed(out_path, **blobs)
    print("wrote", out_path, len(blobs), "arrays", os.path.getsize(out_path), "bytes")


def main():
    if len(sys.argv) > 1 and sys.argv[1] == "offset":
        return main_offset()
    out_path = sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "reference_cuda.npz")
    blobs = {}
    for name, case in cases.all_cases():
        feat, rois, grad = cases.make_inputs(case)
        f, r, g = feat.cuda(), rois.cuda(), grad.cuda()
        kw = dict(spatial_scale=case["spatial_scale"], sampling_ratio=case["sampling_ratio"],
                  aligned=case["aligned"], order=case["order"])
        if case.get("affine_only"):
            blobs[name + "/fwd"] = to_np(ref.forward(f, r, case["out_size"], case["kind"], affine=True, **kw))
            continue
        fwd = ref.forward(f, r, case["out_size"], case["kind"], **kw)
        bwd = ref.backward(g, r, feat.shape, case["kind"], **kw)
        blobs[name + "/fwd"] = to_np(fwd)
        blobs[name + "/bwd"] = to_np(bwd)
        if case["kind"] == cases.KIND_ROTATED and case["order"] == 1:
            # affine_* must equal roi_align_rotated_* forward for orders 0/1
            aff = ref.forward(f, r, case["out_size"], case["kind"], affine=True, **kw)
            assert torch.equal(aff.view(torch.int16) if aff.dtype == torch.float16 else aff,
                               fwd.view(torch.int16) if fwd.dtype == torch.float16 else fwd), name
    np.savez_compressed(out_path, **blobs)
    print("wrote", out_path, len(blobs), "arrays", os.path.getsize(out_path), "bytes")


if __name__ == "__main__":
    main()
