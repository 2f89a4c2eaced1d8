"""CPU-only checks of the drop-in boundary: the shared library loads without a GPU, exports every symbol that
include/callaghan_b200.h declares (and nothing declared is missing from the ctypes table), the configuration helpers
that need no device agree with the oracle's arena layout, and creating a context without a device fails loudly
instead of falling back."""
import ctypes as C
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def _declared():
    text = (ROOT / "include" / "callaghan_b200.h").read_text()
    return sorted(set(re.findall(r"B200_API\s+[\w\s\*]+?\b(b200_\w+)\s*\(", text)))


def test_header_library_and_binding_agree():
    from callaghandev.ml_b200 import _lib

    lib = _lib.load()
    names = _declared()
    assert len(names) >= 60
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in the header but not exported by the library"
        assert n in _lib.PROTOTYPES, f"{n} is declared in the header but has no ctypes prototype"
    assert sorted(_lib.PROTOTYPES) == names, "ctypes table names a symbol the header does not declare"


def test_no_device_means_error_not_fallback():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    from callaghandev.ml_b200 import B200Error, CudaB200AccelerationManager

    with pytest.raises(B200Error):
        CudaB200AccelerationManager(0)


def test_layout_helpers_match_oracle(oracle):
    from callaghandev.ml_b200 import _lib
    from lmutil import lm_config

    lib = _lib.load()
    for cfg in (lm_config(vocab=200, d=64, H=4, L=2, f=128), lm_config(F=5, O=1, d=256, H=8, L=4, f=1024, discrete=False, loss="mse"),
                lm_config(vocab=13, d=8, H=2, L=1, f=16, align=1), lm_config(vocab=32000, d=1024, H=16, L=12, f=4096)):
        c = _lib.LMConfig()
        for name, _ in _lib.LMConfig._fields_:
            setattr(c, name, getattr(cfg, name))
        assert lib.b200_lm_param_count(C.byref(c)) == oracle.lm_param_count(cfg)
        got = []
        for i in range(lib.b200_lm_tensor_count(C.byref(c))):
            off, r, k = C.c_int64(), C.c_int32(), C.c_int32()
            assert lib.b200_lm_tensor_info(C.byref(c), i, C.byref(off), C.byref(r), C.byref(k)) == 0
            got.append((off.value, r.value, k.value))
        assert got == oracle.lm_tensors(cfg)
    bad = _lib.LMConfig()
    assert lib.b200_lm_param_count(C.byref(bad)) == -1


def test_parameter_counts_of_baseline_configs(oracle):
    """Unpadded parameter counts quoted for the benchmark configs: c1 92 744, c3 3 160 833, c4 27 114 304, c5 216 722 688."""
    from lmutil import lm_config

    assert oracle.lm_param_count(lm_config(vocab=200, d=64, H=4, L=2, f=128, align=1)) == 92744
    assert oracle.lm_param_count(lm_config(F=5, O=1, d=256, H=8, L=4, f=1024, discrete=False, loss="mse", align=1)) == 3160833
    assert oracle.lm_param_count(lm_config(vocab=8000, d=512, H=8, L=6, f=2048, align=1)) == 27114304
    assert oracle.lm_param_count(lm_config(vocab=32000, d=1024, H=16, L=12, f=4096, align=1)) == 216722688


def test_split_sequences_covers_batch():
    from callaghandev.ml_b200 import split_sequences

    for n in (0, 1, 7, 256):
        for world in (1, 2, 3, 8):
            spans = [split_sequences(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert max(h - l for l, h in spans) - min(h - l for l, h in spans) <= 1


def test_communicator_cta_limit_is_validated_without_a_device():
    """b200_dp_set_nccl_max_ctas only records the limit for communicators created later: it needs neither a GPU nor NCCL."""
    from callaghandev.ml_b200 import _lib

    lib = _lib.load()
    assert lib.b200_dp_set_nccl_max_ctas(-1) == _lib.ERR_INVALID_ARG
    assert lib.b200_dp_set_nccl_max_ctas(0) == _lib.OK   # 0: leave the choice to NCCL
    assert lib.b200_dp_set_nccl_max_ctas(16) == _lib.OK  # back to the default
