"""Child process of tests/test_gpu_full_size.py: runs tests/full_size_suite.py on the REFERENCE's own CUDA library
(oracle/_ref/libgs_ref.so, its unmodified sources compiled for sm_100) and writes the results to an .npz file.
A separate process because the reference's library and this repository's TorchScript library register the same
class names.  Usage: python tests/ref_runner.py <libgs_ref.so> <out.npz>"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

if __name__ == "__main__":
    lib, out_path = sys.argv[1], sys.argv[2]
    import full_size_suite as suite
    torch.cuda.set_device(0)
    torch.classes.load_library(lib)
    indptr, indices = suite.make_graph(torch.device("cuda", 0))
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    res = suite.run(torch.classes.gs_classes.Graph, torch, indptr, indices)
    np.savez(out_path, **res)
