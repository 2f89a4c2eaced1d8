"""The allocation-free LayerNorm backward (b200_LayerNormBackward_noalloc), called through the C ABI with device
pointers, against the CPU oracle (LayerNormBackward, AccelerationCPU.cs:1516-1564) and against the ordinary entry
point b200_LayerNormBackward on the same data.

Who needs it: a caller whose device memory is entirely owned by its own pool (here: torch's caching allocator stands
in for such a host framework), or a step loop that cannot tolerate the device-wide synchronisation of a driver
allocation.  The entry point therefore takes caller-owned device buffers and keeps its reduction scratch in a fixed
array inside the library.  Two calls in a row with different shapes check that what the first call left in that shared
scratch cannot leak into the second.  Collected last on purpose (file name), and self-contained so that it also passes
alone in a fresh process.
"""
import ctypes as C

import numpy as np
import pytest

from conftest import assert_close
from oracle import pt_matrix, pt_positive_vector, pt_vector

pytestmark = pytest.mark.gpu


def _run_noalloc(lib, torch, dout, x, gamma, mean, var, eps=1e-5):
    dev = torch.device("cuda", 0)
    t = {k: torch.from_numpy(np.ascontiguousarray(v)).to(dev) for k, v in dict(dout=dout, x=x, gamma=gamma, mean=mean, var=var).items()}
    rows, feat = dout.shape
    dx = torch.full((rows, feat), float("nan"), device=dev)
    dg = torch.full((feat,), float("nan"), device=dev)
    db = torch.full((feat,), float("nan"), device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    rc = lib.b200_LayerNormBackward_noalloc(C.c_void_p(stream), C.c_void_p(t["dout"].data_ptr()), C.c_void_p(t["x"].data_ptr()),
                                            C.c_void_p(t["gamma"].data_ptr()), C.c_void_p(t["mean"].data_ptr()), C.c_void_p(t["var"].data_ptr()),
                                            rows, feat, eps, C.c_void_p(dx.data_ptr()), C.c_void_p(dg.data_ptr()), C.c_void_p(db.data_ptr()))
    torch.cuda.synchronize(dev)
    return rc, dx.cpu().numpy(), dg.cpu().numpy(), db.cpu().numpy()


def test_noalloc_layernorm_backward_matches_regular_entry_point(oracle):
    import torch

    from callaghandev.ml_b200 import GEMM_FP32_SIMT, CudaB200AccelerationManager, _lib

    torch.cuda.set_device(0)
    lib = _lib.load()
    mgr = CudaB200AccelerationManager(0, GEMM_FP32_SIMT)
    try:
        # first call: many rows (all 296 partial rows of the built-in scratch are used); second call: few rows and the
        # widest supported row, so most of the scratch still holds the first call's partial sums
        for rows, feat, seed in ((2000, 512, 1), (37, 1024, 5)):
            x, g, b, dout = pt_matrix(rows, feat, seed), pt_positive_vector(feat, seed + 1), pt_vector(feat, seed + 2), pt_matrix(rows, feat, seed + 3)
            _, mean, var, norm = mgr.LayerNormForward(x, g, b)
            e_dx, e_dg, e_db = mgr.LayerNormBackward(dout, norm, g, x, mean, var)
            rc, dx, dg, db = _run_noalloc(lib, torch, dout, x, g, mean, var)
            assert rc == 0
            assert_close(e_dx, dx, 1e-5, "dInput")       # same row kernel: the tolerance of the other LayerNorm tests
            assert_close(e_dg, dg, 3e-5, "dGamma")       # column sums are added in a different block order
            assert_close(e_db, db, 3e-5, "dBeta")
            # and against the CPU oracle itself, so that a fault shared by the two device entry points cannot pass
            _, o_mean, o_var, o_norm = oracle.LayerNormForward(x, g, b)
            o_dx, o_dg, o_db = oracle.LayerNormBackward(dout, o_norm, g, x, o_mean, o_var)
            assert_close(o_dx, dx, 1e-5, "dInput vs oracle")
            assert_close(o_dg, dg, 3e-5, "dGamma vs oracle")
            assert_close(o_db, db, 3e-5, "dBeta vs oracle")
        # sizes beyond the built-in scratch are refused with a status code (and a message on stderr), nothing is launched
        x = np.zeros((4, 2048), np.float32)
        rc, dx, _, _ = _run_noalloc(lib, torch, x, x, np.ones(2048, np.float32), np.zeros(4, np.float32), np.ones(4, np.float32))
        assert rc == _lib.ERR_OUT_OF_RANGE and np.isnan(dx).all()
        x = np.zeros((4, 6), np.float32)
        rc, _, _, _ = _run_noalloc(lib, torch, x, x, np.ones(6, np.float32), np.zeros(4, np.float32), np.ones(4, np.float32))
        assert rc == _lib.ERR_UNSUPPORTED
    finally:
        mgr.Dispose()
