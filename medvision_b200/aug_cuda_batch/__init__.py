from .base import BatchCudaAugBase
from .aug_spatial import (BatchCudaResize, BatchCudaRandomAffine, BatchCudaRandomScale, BatchCudaRandomShift,
                          BatchCudaRandomRotate, BatchCudaRandomElasticDeformation, BatchCudaCropRandomWithAffine, BatchCudaCropCenterWithAffine,
                          BatchCudaCropForegroundWithAffine, BatchCudaCropDetWithAffine,
                          BatchCudaCropFirstDetWithAffine)

__all__ = ['BatchCudaAugBase', 'BatchCudaResize', 'BatchCudaRandomAffine', 'BatchCudaRandomScale',
           'BatchCudaRandomShift', 'BatchCudaRandomRotate', 'BatchCudaRandomElasticDeformation', 'BatchCudaCropRandomWithAffine',
           'BatchCudaCropCenterWithAffine', 'BatchCudaCropForegroundWithAffine', 'BatchCudaCropDetWithAffine',
           'BatchCudaCropFirstDetWithAffine']
