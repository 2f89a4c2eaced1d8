"""The data-parallel step protocol on CPU ranks (host threads), healthy and with injected failures.

The code under test is the product's own `dp_train_step` (callaghandev/ml_b200/csrc/dp_protocol.h) -- the function the
GPU build runs with the resident trainer as engine and NCCL as transport -- compiled here with a toy engine and an
in-memory transport (tests/dp_protocol_sim.cpp).  No GPU is involved and nothing is made to fault: a rank "dies" by
never joining the step, an engine "fails" by returning an error code, a shard "goes non-finite" by holding an infinity.
The rules checked are the reference's, carried over to several ranks (TransformerTrainer.cs:298-307: a failure drops the
batch and zeroes every gradient; :316-320: a non-finite gradient norm zeroes the gradients and skips the update).
"""
import ctypes as C
import subprocess
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
HEALTHY, ENGINE_ERROR, RANK_ABSENT, NONFINITE_SHARD, EMPTY_SHARD, OUT_OF_ORDER = range(6)
DP_OK, DP_ERR_PEER, DP_ERR_TIMEOUT, DP_ERR_COMM, DP_ERR_PROTOCOL = 0, 101, 102, 103, 104
TOTAL, RANGES = 1000, 4


@pytest.fixture(scope="module")
def sim(tmp_path_factory):
    so = tmp_path_factory.mktemp("dpsim") / "libdpsim.so"
    subprocess.run(["g++", "-O1", "-std=c++17", "-shared", "-fPIC", "-pthread", "-o", str(so), str(ROOT / "tests" / "dp_protocol_sim.cpp")], check=True)
    return C.CDLL(str(so))


def run(sim, world, scenario, bad_rank=1, deadline_ms=2000):
    rc, valid, skipped = (np.zeros(world, np.int32) for _ in range(3))
    loss, norm, ms = (np.zeros(world, np.float32) for _ in range(3))
    w, g = np.zeros((world, TOTAL), np.float32), np.zeros((world, TOTAL), np.float32)
    p = lambda a, t: a.ctypes.data_as(C.POINTER(t))
    sim.dp_sim_run(world, TOTAL, RANGES, scenario, bad_rank, deadline_ms, p(rc, C.c_int32), p(valid, C.c_int32), p(loss, C.c_float), p(norm, C.c_float),
                   p(ms, C.c_float), p(w, C.c_float), p(g, C.c_float), p(skipped, C.c_int32))
    return dict(rc=rc, valid=valid, loss=loss, norm=norm, ms=ms, w=w, g=g, skipped=skipped)


def w0():
    return np.float32(0.01) * (np.arange(TOTAL) % 17).astype(np.float32)


def local_grad(rank):
    i = np.arange(TOTAL)
    return (np.float32(0.001) * ((i * 7 + rank * 13) % 29).astype(np.float32) - np.float32(0.01)).astype(np.float32)


@pytest.mark.parametrize("world", [2, 4])
def test_healthy_step_equals_the_single_process_sum(sim, world):
    r = run(sim, world, HEALTHY)
    assert (r["rc"] == DP_OK).all()
    valid = sum(range(1, world + 1))
    assert (r["valid"] == valid).all()
    np.testing.assert_allclose(r["loss"], sum(1.5 * (k + 1) for k in range(world)) / valid, rtol=1e-6)
    g = sum(local_grad(k).astype(np.float64) for k in range(world)) / valid
    norm = np.sqrt((g * g).sum())
    g = g * (0.05 / norm if norm > 0.05 else 1.0)
    for k in range(world):
        np.testing.assert_allclose(r["g"][k], g, rtol=2e-5, atol=1e-8)
        np.testing.assert_allclose(r["w"][k], w0() - 0.1 * g, rtol=1e-5, atol=1e-7)
        assert np.array_equal(r["g"][k], r["g"][0]) and np.array_equal(r["w"][k], r["w"][0]), "every rank must end with identical bits"


def test_a_rank_whose_pass_fails_drops_the_step_everywhere(sim):
    """Rank 1's engine returns an error after announcing one range.  It still issues every collective, the failure
    travels in the scalar reduction, and every rank discards the step: gradients zero, weights untouched, nobody blocks."""
    r = run(sim, 3, ENGINE_ERROR, bad_rank=1, deadline_ms=5000)
    assert r["rc"].tolist() == [DP_ERR_PEER, 77, DP_ERR_PEER]
    assert (r["ms"] < 1000).all(), "the error must arrive through the protocol, not through the deadline"
    for k in range(3):
        assert not r["g"][k].any(), "gradients are zeroed on every rank (TransformerTrainer.cs:298-307)"
        assert np.array_equal(r["w"][k], w0()), "weights are untouched"


def test_a_rank_that_never_joins_times_its_peers_out(sim):
    """Rank 2 dies before its first collective.  Its peers give up at the deadline instead of blocking for ever, abort
    the transport and discard the step."""
    r = run(sim, 3, RANK_ABSENT, bad_rank=2, deadline_ms=300)
    assert r["rc"][2] == -1  # never ran
    assert sorted(r["rc"][:2].tolist()) in ([DP_ERR_TIMEOUT, DP_ERR_TIMEOUT], [DP_ERR_TIMEOUT, DP_ERR_COMM])  # the second may see the first one's abort
    assert (r["ms"][:2] >= 250).all() and (r["ms"][:2] < 2000).all()
    for k in range(2):
        assert not r["g"][k].any() and np.array_equal(r["w"][k], w0())


def test_a_non_finite_shard_makes_every_rank_skip_identically(sim):
    """One rank's gradients hold an infinity.  After the reduction every rank holds it, computes a non-finite norm,
    zeroes its gradients and skips the update -- the same decision everywhere without any extra exchange."""
    r = run(sim, 4, NONFINITE_SHARD, bad_rank=0)
    assert (r["rc"] == DP_OK).all() and (r["skipped"] == 1).all()
    assert not np.isfinite(r["norm"]).any()
    for k in range(4):
        assert not r["g"][k].any() and np.array_equal(r["w"][k], w0())


def test_a_rank_with_nothing_to_train_still_issues_every_collective(sim):
    """An empty or all-invalid shard announces no range itself; the protocol completes the sequence for it, and the other
    ranks' step equals the step without that rank."""
    world = 3
    r = run(sim, world, EMPTY_SHARD, bad_rank=1)
    assert (r["rc"] == DP_OK).all()
    valid = 1 + 3
    assert (r["valid"] == valid).all()
    g = (local_grad(0).astype(np.float64) + local_grad(2)) / valid
    norm = np.sqrt((g * g).sum())
    g = g * (0.05 / norm if norm > 0.05 else 1.0)
    for k in range(world):
        np.testing.assert_allclose(r["g"][k], g, rtol=2e-5, atol=1e-8)
        assert np.array_equal(r["w"][k], r["w"][0])


def test_an_out_of_order_announcement_is_a_protocol_error(sim):
    r = run(sim, 2, OUT_OF_ORDER, bad_rank=0, deadline_ms=300)
    assert r["rc"][0] == DP_ERR_PROTOCOL
    assert r["rc"][1] in (DP_ERR_TIMEOUT, DP_ERR_COMM)
    for k in range(2):
        assert not r["g"][k].any() and np.array_equal(r["w"][k], w0())


def test_shard_bounds_through_the_library():
    """b200_dp_shard needs no GPU: contiguous shards that cover the batch, the first n % world ranks one longer."""
    from callaghandev.ml_b200 import _lib

    lib = _lib.load()
    for n, world in ((13, 4), (3, 8), (0, 2), (256, 8)):
        prev = 0
        sizes = []
        for r in range(world):
            lo, hi = C.c_int32(), C.c_int32()
            assert lib.b200_dp_shard(n, r, world, C.byref(lo), C.byref(hi)) == 0
            assert lo.value == prev and hi.value >= lo.value
            sizes.append(hi.value - lo.value)
            prev = hi.value
        assert prev == n and max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)
    assert lib.b200_dp_shard(5, 2, 2, C.byref(lo), C.byref(hi)) != 0
