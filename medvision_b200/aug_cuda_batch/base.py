"""Base class of the batched CUDA augmentations.

Same protocol as medvision/aug_cuda_batch/base.py: a transform is a callable on a ``result``
dict (``img_dim``, ``img_fields`` / ``seg_fields`` naming (B, C, [D,] H, W) CUDA tensors, ...);
``forward`` draws the parameters with numpy's / random's global generators in the reference's
order (so a seeded run picks the same parameters), applies them to every field, stores them
under ``<ClassName>_params`` and appends to ``history`` / ``time`` / ``memory``;
``backward`` (for transforms with ``canBackward``) applies the inverse transform.
"""
import random
import time
from datetime import datetime
from typing import Iterable, List, Tuple, Union

import numpy as np
import torch


class BatchCudaAugBase(object):
    def __init__(self):
        self.p = 0.
        self.latitude = 1.0
        self.always = False
        self.dim = None
        self.params = None
        self.isForwarding = None
        self.name = self.__class__.__name__
        self.key_name = self.name + '_params'

    def __repr__(self):
        return self.__class__.__name__ + '()'

    @property
    def canBackward(self):
        return False

    @property
    def repeats(self):
        return 1

    @staticmethod
    def get_range(val_range, bias=0, always_pos=False):
        if isinstance(val_range, (int, float)):
            val_range = [0, val_range] if always_pos else [-val_range, val_range]
        assert isinstance(val_range, (list, tuple)) and len(val_range) == 2
        assert val_range[1] >= val_range[0]
        return bias + np.random.uniform(*val_range)

    @staticmethod
    def to_tuple(value: Union[int, float, Iterable[int], Iterable[float]], length: int = 1) \
            -> Union[Tuple[int], Tuple[float]]:
        try:
            iter(value)
            value = tuple(value)
        except TypeError:
            value = length * (value,)
        assert len(value) == length, f'Dimension not match. Required is {length}D but value is {len(value)}D'
        return value

    def _init_params(self, result):
        self.dim = self.dim if self.dim else result['img_dim']
        self.img_type = result['img'].dtype
        self.array_shape = tuple(result['img'].shape)
        self.image_axes = tuple(range(2, self.dim + 2))
        self.batch = self.array_shape[0]
        self.channels = self.array_shape[1]
        self.image_shape = self.array_shape[2:]
        self.params = None

    def _forward_params(self, result: dict):
        pass

    def _backward_params(self, result: dict):
        pass

    def setLatitude(self, val):
        self.latitude = val

    def getLatitude(self):
        return self.latitude

    def apply_to_img(self, result: dict):
        pass

    def apply_to_cls(self, result: dict):
        pass

    def apply_to_seg(self, result: dict):
        pass

    def apply_to_det(self, result: dict):
        pass

    def _pre_forward(self, result: dict):
        assert isinstance(result, dict), f'A dict is required but got a {type(result)}!'
        self._debug_ = result.get('_debug_', False)
        self._tic_ = time.time()
        return result

    def _forward(self, result: dict):
        self.isForwarding = True
        assert self.always or self.p > 0., f'self.always={self.always} or self.p={self.p} is needed.'
        if self.always or random.random() <= self.p * self.latitude:
            self.params = None
            self._forward_params(result)
            self.apply_to_img(result)
            self.apply_to_cls(result)
            self.apply_to_seg(result)
            self.apply_to_det(result)
        return result

    def _post_forward(self, result: dict):
        assert isinstance(result, dict), f'A dict is required but got a {type(result)}!'
        result.setdefault('history', [])
        result.setdefault('time', [])
        result.setdefault('memory', [])
        start = datetime.fromtimestamp(self._tic_).strftime('%H:%M:%S.%f')
        # same unit as the reference's record (its divisor includes a factor 8)
        mem = torch.cuda.max_memory_allocated() / 1024 / 1024 / 8 if torch.cuda.is_available() else 0.0
        result['history'].append(self.name)
        result['memory'].append(f"{self.name}-{mem:.02f}MB")
        result['time'].append(f"{self.name}-{start}-{time.time() - self._tic_:.03f}s")
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

    def _pre_backward(self, result: dict):
        time_cost = result['time'].pop()
        last = result['history'].pop()
        assert self.name in time_cost, f'{self.name} {time_cost}'
        assert last == self.name, f'require params to be {self.name}, but the last is {last}'
        return result

    def _backward(self, result: dict):
        assert isinstance(result, dict)
        self.isForwarding = False
        if self.canBackward:
            self.params = None
            self._backward_params(result)
            if self.params is not None:
                self.apply_to_img(result)
                self.apply_to_cls(result)
                self.apply_to_seg(result)
                self.apply_to_det(result)
        return result

    def _post_backward(self, result: dict):
        return result

    def backward(self, result):
        return self._post_backward(self._backward(self._pre_backward(result)))

    def __call__(self, result: Union[dict, List[dict]], forward=True):
        if forward:
            if self.repeats > 1:
                return self.multi_forward(result)
            return self.forward(result)
        raise NotImplementedError
