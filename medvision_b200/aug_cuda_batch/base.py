"""Base class of the batched CUDA augmentations.

The protocol is the one of medvision/aug_cuda_batch/base.py (names, ``result`` keys and the order
of the random draws are the interface a pipeline relies on; the bodies are this package's own):

* a transform is a callable on a ``result`` dict: ``img_dim``, the fields named by
  ``img_fields`` / ``seg_fields`` as (B, C, [D,] H, W) CUDA tensors, ...;
* ``forward`` decides with ONE ``random.random()`` draw (skipped when ``always``) whether the
  transform fires, then lets the subclass draw its parameters (``_forward_params``, numpy's global
  generator) and apply them field family by field family; it logs itself under ``history``,
  ``time`` and ``memory``;
* ``backward`` pops that log entry and, for a transform with ``canBackward``, applies the inverse
  parameters (``_backward_params``) through the same ``apply_to_*`` hooks.
"""
import random
import time
from datetime import datetime
from typing import Iterable, List, Tuple, Union

import numpy as np
import torch

# field families, in the order the hooks run
_HOOKS = ('apply_to_img', 'apply_to_cls', 'apply_to_seg', 'apply_to_det')
_LOG_KEYS = ('history', 'time', 'memory')


class BatchCudaAugBase(object):
    def __init__(self):
        cls_name = type(self).__name__
        self.name, self.key_name = cls_name, cls_name + '_params'
        self.p, self.latitude, self.always = 0., 1.0, False
        self.dim = self.params = self.isForwarding = None

    def __repr__(self):
        return f'{type(self).__name__}()'

    # ---- capabilities ---------------------------------------------------------------------
    @property
    def canBackward(self):
        return False

    @property
    def repeats(self):
        return 1

    def setLatitude(self, val):
        self.latitude = val

    def getLatitude(self):
        return self.latitude

    # ---- parameter helpers ------------------------------------------------------------------
    @staticmethod
    def get_range(val_range, bias=0, always_pos=False):
        """One uniform draw: a number r stands for [-r, r] (or [0, r] with ``always_pos``), a pair is
        taken as it is; ``bias`` is added to the draw."""
        if not isinstance(val_range, (list, tuple)):
            assert isinstance(val_range, (int, float))
            val_range = (0 if always_pos else -val_range, val_range)
        lo, hi = val_range  # a pair, nothing else
        assert hi >= lo
        return bias + np.random.uniform(lo, hi)

    @staticmethod
    def to_tuple(value: Union[int, float, Iterable[int], Iterable[float]], length: int = 1) \
            -> Union[Tuple[int], Tuple[float]]:
        """Scalar -> ``length`` copies of it; iterable -> tuple of it, which must have ``length`` items."""
        value = tuple(value) if isinstance(value, Iterable) else (value,) * length
        assert len(value) == length, f'Dimension not match. Required is {length}D but value is {len(value)}D'
        return value

    def _init_params(self, result):
        """Shape bookkeeping the subclasses read: taken from ``result['img']`` (B, C, *spatial)."""
        img = result['img']
        if not self.dim:
            self.dim = result['img_dim']
        self.img_type, self.array_shape = img.dtype, tuple(img.shape)
        self.batch, self.channels = self.array_shape[:2]
        self.image_shape = self.array_shape[2:]
        self.image_axes = tuple(range(2, 2 + self.dim))
        self.params = None

    # ---- hooks of the subclasses ------------------------------------------------------------
    def _forward_params(self, result: dict):
        pass

    def _backward_params(self, result: dict):
        pass

    def apply_to_img(self, result: dict):
        pass

    def apply_to_cls(self, result: dict):
        pass

    def apply_to_seg(self, result: dict):
        pass

    def apply_to_det(self, result: dict):
        pass

    def _apply_all(self, result):
        for hook in _HOOKS:
            getattr(self, hook)(result)

    # ---- forward ---------------------------------------------------------------------------
    def _pre_forward(self, result: dict):
        assert isinstance(result, dict), f'A dict is required but got a {type(result)}!'
        self._tic_ = time.time()
        self._debug_ = result.get('_debug_', False)
        return result

    def _fires(self):
        assert self.always or self.p > 0., f'self.always={self.always} or self.p={self.p} is needed.'
        return self.always or random.random() <= self.p * self.latitude

    def _forward(self, result: dict):
        self.isForwarding = True
        if self._fires():
            self.params = None
            self._forward_params(result)
            self._apply_all(result)
        return result

    def _post_forward(self, result: dict):
        assert isinstance(result, dict), f'A dict is required but got a {type(result)}!'
        for key in _LOG_KEYS:
            result.setdefault(key, [])
        took = time.time() - self._tic_
        began = datetime.fromtimestamp(self._tic_).strftime('%H:%M:%S.%f')
        # the reference logs the allocator's peak divided by 1024 * 1024 * 8 under the label "MB"; kept as is
        peak = torch.cuda.max_memory_allocated() / (1024 * 1024 * 8) if torch.cuda.is_available() else 0.0
        result['history'].append(self.name)
        result['time'].append(f"{self.name}-{began}-{took:.03f}s")
        result['memory'].append(f"{self.name}-{peak:.02f}MB")
        return result

    def forward(self, result: dict):
        return self._post_forward(self._forward(self._pre_forward(result)))

    def multi_forward(self, result: dict):
        """``repeats`` crops per image.  The reference concatenates ``repeats`` copies of every
        field and crops each copy once (medvision/aug_cuda_batch/base.py:175-180); here the
        images stay as they are and the rois of repeat r point at image (r*B + b) % B, which
        gives the same output, in the same order, without the copies."""
        assert self.repeats > 1
        return self.forward(result)

    # ---- backward (inverse transform of test-time augmentation) ---------------------------------
    def _pre_backward(self, result: dict):
        stamp, last = result['time'].pop(), result['history'].pop()
        assert last == self.name, f'require params to be {self.name}, but the last is {last}'
        assert self.name in stamp, f'{self.name} {stamp}'
        return result

    def _backward(self, result: dict):
        assert isinstance(result, dict)
        self.isForwarding = False
        if not self.canBackward:
            return result
        self.params = None
        self._backward_params(result)
        if self.params is not None:  # None: the forward pass did not fire on this result
            self._apply_all(result)
        return result

    def _post_backward(self, result: dict):
        return result

    def backward(self, result):
        return self._post_backward(self._backward(self._pre_backward(result)))

    def __call__(self, result: Union[dict, List[dict]], forward=True):
        if not forward:
            raise NotImplementedError
        return self.multi_forward(result) if self.repeats > 1 else self.forward(result)
