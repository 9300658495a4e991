from .base import CudaAugBase
from .aug_spatial import (CudaResize, CudaRandomAffine, CudaRandomScale, CudaRandomShift, CudaRandomRotate,
                          CudaRandomElasticDeformation, CudaCropRandomWithAffine, CudaCropCenterWithAffine,
                          CudaCropFirstDetWithAffine)
from .aug_testtime import CudaPatches

__all__ = ['CudaAugBase', 'CudaResize', 'CudaRandomAffine', 'CudaRandomScale', 'CudaRandomShift', 'CudaRandomRotate',
           'CudaRandomElasticDeformation', 'CudaCropRandomWithAffine', 'CudaCropCenterWithAffine',
           'CudaCropFirstDetWithAffine', 'CudaPatches']
