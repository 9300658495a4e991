from .aug_testtime import CudaPatches

__all__ = ['CudaPatches']
