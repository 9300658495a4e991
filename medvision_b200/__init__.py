"""medvision-b200: B200 (sm_100a) RoI Align / RoI Align Rotated / affine resampling.

Drop-in for the resampling path of MedVision: ``medvision_b200.ops`` mirrors
``medvision.ops`` (RoIAlign, RoIAlignRotated) and ``medvision.ops.cuda_fun_tools``
(affine_2d, affine_3d); ``medvision_b200._C`` mirrors the ten functions of the reference's
compiled extension on that path.  There is no CPU implementation.
"""
__version__ = "0.1.0"
