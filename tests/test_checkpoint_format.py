"""The reference's checkpoint directory (LanguageModel.Save / Load, LanguageModel.cs:706-869), written and read from the
flat parameter arena.  The checks use an INDEPENDENT reader and writer restated here from the C# calls -- BinaryWriter
little-endian primitives in the order of Save (:737-765), WriteMatrix = int32 rows, int32 cols, floats (:840-853),
WriteVector = int32 length, floats (:854-863), WriteAttention = WQ WK WV WO BiasQ BiasK BiasV BiasO (:864-868) -- so a
mistake in the module under test cannot cancel itself out.  No GPU is needed: the arena layout comes from the library's
b200_lm_tensor_info, which is pure host code."""
import ctypes as C
import io
import json
import struct

import numpy as np
import pytest

from callaghandev.ml_b200 import _lib, make_config
from callaghandev.ml_b200.checkpoint import load_reference_checkpoint, save_reference_checkpoint

CONFIG_KEYS = ["VocabSize", "MaxSequenceLength", "EmbeddingDim", "NumHeads", "NumLayers", "FeedForwardDim", "UseDecoderOnly", "FFNActivationType",
               "AccelerationType", "AccelerationDeviceId", "L2RegulationLamda", "GradientClippingThreshold", "DataType", "InputFeatureDim", "OutputDim",
               "CostFunction", "ActivationDistribution"]  # LanguageModel.cs:710-729, in that order


def table(cfg):
    lib = _lib.load()
    out = []
    for i in range(lib.b200_lm_tensor_count(C.byref(cfg))):
        off, r, c = C.c_int64(), C.c_int32(), C.c_int32()
        lib.b200_lm_tensor_info(C.byref(cfg), i, C.byref(off), C.byref(r), C.byref(c))
        out.append((off.value, r.value, c.value))
    return out, int(lib.b200_lm_param_count(C.byref(cfg)))


def csharp_reader(blob, discrete, L):
    """What LanguageModel.Load does with weights.bin, tensor by tensor; returns the list of arrays in file order."""
    f = io.BytesIO(blob)
    rd_i = lambda: struct.unpack("<i", f.read(4))[0]
    rd_m = lambda: (lambda r, c: np.frombuffer(f.read(4 * r * c), "<f4").reshape(r, c))(rd_i(), rd_i())
    rd_v = lambda: np.frombuffer(f.read(4 * rd_i()), "<f4")
    assert struct.unpack("<?", f.read(1))[0] == discrete
    out = [rd_m()] if discrete else [rd_m(), rd_v()]
    for _ in range(L):
        out += [rd_m() for _ in range(4)] + [rd_v() for _ in range(8)]
    out += [rd_m(), rd_v()]
    assert f.read() == b"", "nothing may follow the output bias"
    return out


def csharp_writer(arrays, discrete):
    """What LanguageModel.Save writes for the given tensors (2-D = WriteMatrix, 1-D = WriteVector)."""
    f = io.BytesIO()
    f.write(struct.pack("<?", discrete))
    for a in arrays:
        f.write(struct.pack("<ii", *a.shape) if a.ndim == 2 else struct.pack("<i", a.size))
        f.write(np.ascontiguousarray(a, "<f4").tobytes())
    return f.getvalue()


@pytest.mark.parametrize("kind", ["text", "regression"])
def test_written_directory_is_the_reference_format(tmp_path, kind):
    rng = np.random.default_rng(1)
    if kind == "text":
        cfg = make_config(vocab_size=37, embedding_dim=16, num_heads=4, num_layers=2, ffn_dim=24, ffn_activation="Relu")
    else:
        cfg = make_config(input_feature_dim=5, output_dim=1, embedding_dim=16, num_heads=2, num_layers=1, ffn_dim=20, ffn_activation="Tanh", discrete=False, loss="mse")
    tensors, total = table(cfg)
    P = np.zeros(total, np.float32)
    for off, r, c in tensors:
        P[off:off + r * c] = rng.normal(0, 1, r * c).astype(np.float32) * np.float32(10.0) ** rng.integers(-6, 3)
    m, v = rng.normal(0, 1e-3, total).astype(np.float32), rng.uniform(0, 1e-6, total).astype(np.float32)
    save_reference_checkpoint(tmp_path, cfg, tensors, P, 64, {"GradientClippingThreshold": 1.0, "L2RegulationLamda": 1e-4}, adam=(m, v, 17))

    conf = json.loads((tmp_path / "config.json").read_text())
    assert list(conf) == CONFIG_KEYS
    assert conf["EmbeddingDim"] == 16 and conf["MaxSequenceLength"] == 64 and conf["UseDecoderOnly"] is True
    assert conf["DataType"] == (0 if kind == "text" else 1) and conf["FFNActivationType"] == (3 if kind == "text" else 2)

    L, n0 = cfg.num_layers, 1 if cfg.discrete else 2
    got = csharp_reader((tmp_path / "weights.bin").read_bytes(), bool(cfg.discrete), L)
    # arena tensors that live in weights.bin, in file order: the first 12 of each block's 16 (the FFN goes to JSON)
    want = tensors[:n0] + [t for l in range(L) for t in tensors[n0 + 16 * l:n0 + 16 * l + 12]] + tensors[-2:]
    assert len(got) == len(want)
    for a, (off, r, c) in zip(got, want):
        assert a.size == r * c and np.array_equal(a.reshape(-1), P[off:off + r * c]), "weights.bin must hold the arena's bits"
        assert a.ndim == (2 if r > 1 or (r * c == cfg.embedding_dim * cfg.embedding_dim) else a.ndim)
    d, f = cfg.embedding_dim, cfg.ffn_dim
    shapes = [a.shape for a in got]
    assert shapes[n0:n0 + 12] == [(d, d)] * 4 + [(d,)] * 8 and shapes[-2:] == [(cfg.output_dim, d), (cfg.output_dim,)]
    assert shapes[0] == ((cfg.vocab_size, d) if cfg.discrete else (d, cfg.input_feature_dim))

    for l in range(L):
        net = json.loads((tmp_path / "ffn" / f"ffn_layer_{l}.json").read_text())
        assert list(net) == ["layers", "parameters"] and len(net["layers"]) == 3
        l0, l1, l2 = net["layers"]
        assert (l0["Size"], l0["InputSize"], l1["Size"], l1["InputSize"], l2["Size"], l2["InputSize"]) == (d, 0, f, d, d, f)
        assert l0["Weights"] == [[] for _ in range(d)], "the input layer's float[size, 0] serialises as empty rows"
        assert [x["ActivationType"] for x in net["layers"]] == [0, cfg.ffn_activation, 0]
        for key in ("Activations", "Biases", "Derivatives", "Deltas"):
            assert len(l1[key]) == f
        base = n0 + 16 * l
        for lay, (tw, tb) in ((l1, (tensors[base + 12], tensors[base + 13])), (l2, (tensors[base + 14], tensors[base + 15]))):
            W = np.asarray(lay["Weights"], np.float64).astype(np.float32)  # Newtonsoft parses a double and narrows
            assert np.array_equal(W.reshape(-1), P[tw[0]:tw[0] + tw[1] * tw[2]]), "JSON numbers must read back to the same float32"
            assert np.array_equal(np.asarray(lay["Biases"], np.float64).astype(np.float32), P[tb[0]:tb[0] + tb[1] * tb[2]])
        p = net["parameters"]
        assert p["LayerWidths"] == [d, f, d] and p["LayerActivations"] == [0, cfg.ffn_activation, 0]
        assert p["inputActivationMin"] == [0.0] * d and p["inputActivationMax"] == [1.0] * d  # TransformerBlock.cs:119-121

    cfg2, P2, conf2, adam = load_reference_checkpoint(tmp_path, make_config, table)
    assert [getattr(cfg2, n) for n, _ in _lib.LMConfig._fields_] == [getattr(cfg, n) for n, _ in _lib.LMConfig._fields_]
    assert np.array_equal(P2, P)
    assert adam[2] == 17 and np.array_equal(adam[0], m) and np.array_equal(adam[1], v)


def test_a_directory_written_the_csharp_way_loads(tmp_path):
    """weights.bin assembled by the restated C# writer and FFN files as Newtonsoft lays them out (UTF-8 with a byte-order
    mark, indented, extra members): the loader must fill the arena with exactly those values."""
    rng = np.random.default_rng(2)
    cfg = make_config(vocab_size=11, embedding_dim=8, num_heads=2, num_layers=1, ffn_dim=12, ffn_activation="Leakyrelu")
    d, f, V = 8, 12, 11
    r = lambda *s: rng.normal(0, 0.3, s).astype(np.float32)
    arrays = [r(V, d)] + [r(d, d) for _ in range(4)] + [r(d) for _ in range(8)] + [r(V, d), r(V)]
    (tmp_path / "ffn").mkdir()
    (tmp_path / "weights.bin").write_bytes(csharp_writer(arrays, True))
    conf = dict(zip(CONFIG_KEYS, [V, 32, d, 2, 1, f, True, 4, 1, 0, 0.0, 1.0, 0, 0, 0, 0, 0]))
    (tmp_path / "config.json").write_text(json.dumps(conf, indent=2))
    W1, b1, W2, b2 = r(f, d), r(f), r(d, f), r(d)
    fl = lambda a: [float(x) for x in a]
    lay = lambda size, inp, W, b, act: {"Size": size, "InputSize": inp, "Activations": [0.0] * size, "Biases": fl(b), "Derivatives": [0.0] * size,
                                        "Deltas": [0.0] * size, "Weights": [fl(row) for row in W], "ActivationType": act}
    net = {"layers": [lay(d, 0, np.zeros((d, 0)), np.zeros(d), 0), lay(f, d, W1, b1, 4), lay(d, f, W2, b2, 0)],
           "parameters": {"HuberLossDelta": 1.0, "LayerWidths": [d, f, d], "LayerActivations": [0, 4, 0], "OptimalLearningRate": None}}
    (tmp_path / "ffn" / "ffn_layer_0.json").write_bytes(b"\xef\xbb\xbf" + json.dumps(net, indent=2).encode())
    cfg2, P, _, adam = load_reference_checkpoint(tmp_path, make_config, table)
    assert adam is None and cfg2.ffn_activation == 4 and cfg2.vocab_size == V
    tensors, _ = table(cfg2)
    want = [arrays[0]] + arrays[1:13] + [W1, b1, W2, b2] + arrays[13:]
    for (off, rr, cc), a in zip(tensors, want):
        assert np.array_equal(P[off:off + rr * cc], a.reshape(-1))
    # shape mismatches are refused like ReadMatrixInto does, and a missing FFN file like LoadFeedForwardNetworks
    bad = list(arrays); bad[1] = r(d, d + 1)
    (tmp_path / "weights.bin").write_bytes(csharp_writer(bad, True))
    with pytest.raises(ValueError):
        load_reference_checkpoint(tmp_path, make_config, table)
    (tmp_path / "weights.bin").write_bytes(csharp_writer(arrays, True))
    (tmp_path / "ffn" / "ffn_layer_0.json").unlink()
    with pytest.raises(FileNotFoundError):
        load_reference_checkpoint(tmp_path, make_config, table)
