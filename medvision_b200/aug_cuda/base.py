"""Base class of the single-sample CUDA augmentations.

Same protocol as medvision/aug_cuda/base.py:27-223: a transform is a callable on one ``result``
dict whose image / label fields are (C, [D,] H, W) CUDA tensors (no batch axis), or on a list of
such dicts; ``forward`` draws the parameters with numpy's / random's global generators in the
reference's order, applies them to every field, stores them under ``<ClassName>_params`` and
appends to ``history`` / ``time`` / ``memory``; a transform with ``repeats`` > 1 turns one dict into
``repeats`` dicts; ``backward`` applies the inverse of a transform with ``canBackward``.
"""
import random
import time
from copy import copy
from datetime import datetime
from typing import List, Union

import torch

from ..aug_cuda_batch.base import BatchCudaAugBase


class CudaAugBase(BatchCudaAugBase):
    """Shares the parameter helpers (``get_range``, ``to_tuple``) and the forward / backward
    bookkeeping with the batched base class; differs in the field layout and in list handling."""

    def _init_params(self, result):
        self.dim = self.dim if self.dim else result['img_dim']
        self.img_type = result['img'].dtype
        self.array_shape = tuple(result['img'].shape) if 'img' in result else tuple(result['img_shape'])
        self.image_axes = tuple(range(1, self.dim + 1))
        self.channels = self.array_shape[0]
        self.image_shape = self.array_shape[1:]
        self.params = None

    @staticmethod
    def _copy_result(result: dict) -> dict:
        """A repeat gets its own dict and its own bookkeeping lists; tensors are shared until a
        transform replaces them (the reference deep-copies them, medvision/aug_cuda/base.py:166)."""
        dup = copy(result)
        for key in ('history', 'time', 'memory', 'img_fields', 'seg_fields', 'det_fields'):
            if key in dup:
                dup[key] = list(dup[key])
        return dup

    def multi_forward(self, result_list: Union[List[dict], dict]):
        if self.repeats > 1:
            results = [result_list] if isinstance(result_list, dict) else result_list
            return [self.forward(self._copy_result(r)) for r in results for _ in range(self.repeats)]
        assert isinstance(result_list, list) and self.repeats == 1
        return [self.forward(result) for result in result_list]

    def multi_backward(self, result_list: list):
        return [self.backward(result) for result in result_list]

    def __call__(self, result: Union[dict, List[dict]], forward=True):
        if forward:
            if isinstance(result, dict) and self.repeats == 1:
                return self.forward(result)
            if isinstance(result, list) or self.repeats > 1:
                return self.multi_forward(result)
            raise NotImplementedError
        if isinstance(result, list):
            return self.multi_backward(result)
        return self.backward(result)
