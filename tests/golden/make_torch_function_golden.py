"""Generate tests/golden/torch_function_c1.npz with the reference's OWN torch-function RoIAlign.

Needs the reference checkout (it is loaded by file path because the package's __init__ imports
the compiled extension); run where that checkout exists:

    python tests/golden/make_torch_function_golden.py /path/to/reference
"""
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle.torch_function_path import config1_inputs  # noqa: E402


def main():
    root = sys.argv[1]
    path = os.path.join(root, "medvision", "ops", "pytorch_ops", "roi_align.py")
    spec = importlib.util.spec_from_file_location("ref_torch_function_roi_align", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    feat, rois = config1_inputs(n_rois=16)
    feat.requires_grad_(True)
    out = mod.RoIAlign((7, 7, 7), 1.0, 2)(feat, rois)
    g = torch.Generator().manual_seed(2)
    grad = torch.randn(out.shape, generator=g)
    out.backward(grad)
    # the gradient is sparse: keep its checksum per (sample, channel) and a slab
    np.savez_compressed(os.path.join(HERE, "torch_function_c1.npz"), out=out.detach().numpy(),
                        grad_sum=feat.grad.sum(dim=(2, 3, 4)).numpy(), grad_slab=feat.grad[0, 0, 30:34].numpy())
    print("ok", out.shape)


if __name__ == "__main__":
    main()
