"""The reference's on-disk model format, read and written from the flat parameter arena of the resident trainer.

A directory as LanguageModel.Save lays it out (Transformers/MultiTypeTransformer/LanguageModel.cs:706-765) and
LanguageModel.Load reads it (:769-869):

  config.json        the model shape and run-time enums as a flat JSON object (:710-735)
  weights.bin        BinaryWriter, little endian: one byte UsesDiscreteTokens; a matrix is int32 rows, int32 cols, then
                     rows*cols float32 row-major (WriteMatrix :840-853); a vector is int32 length, then float32s
                     (WriteVector :854-863); order: TokenEmbedding | InputProjection + InputProjectionBias; per layer WQ
                     WK WV WO BiasQ BiasK BiasV BiasO (WriteAttention :864-868), LN1Gamma LN1Beta LN2Gamma LN2Beta;
                     OutputProjection, OutputBias (:737-765)
  ffn/ffn_layer_i.json   each block's feed-forward NeuralNetwork as Newtonsoft JSON of its Data object: "layers" (three
                     Layer objects: Size, InputSize, Activations, Biases, Derivatives, Deltas, Weights as nested arrays,
                     ActivationType) and "parameters" (:671-685; Neural Network/Data.cs:218-236, Layer.cs, Parameters.cs)

so that a model trained here loads in the reference (`LanguageModel.Load`) and the reverse.  The arena holds exactly
these tensors in this order with each block's FFN tensors appended to the block (b200_lm_tensor_info), which makes the
conversion a walk over the tensor table.  The Adam moments and the step index are this library's extension: they go
into `optimizer.bin` beside the reference's files, which the reference ignores.
"""
from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np

# TransformerDataType (Transformers/MultiTypeTransformer/TransformerDataType.cs)
DATA_TEXT, DATA_TS_REGRESSION, DATA_TS_CLASSIFICATION, DATA_SYMBOLIC = 0, 1, 2, 3
# AccelerationType (Neural Network/Enums/AccelerationType.cs): a checkpoint written here says CPU so that any build of the reference can open it
ACCEL_CPU = 0
OPT_MAGIC = b"B200ADAM"


def _data_type(cfg) -> int:
    if cfg.discrete:
        return DATA_TEXT
    return DATA_TS_REGRESSION if cfg.loss_kind == 1 else DATA_TS_CLASSIFICATION


def _layer_tensor_slices(cfg, tensors):
    """tensors = [(offset, rows, cols)] of the arena.  Returns (first, per-layer list of 16, last two)."""
    n0 = 1 if cfg.discrete else 2
    L = cfg.num_layers
    assert len(tensors) == n0 + 16 * L + 2, "tensor table does not match the configuration"
    return tensors[:n0], [tensors[n0 + 16 * l:n0 + 16 * (l + 1)] for l in range(L)], tensors[n0 + 16 * L:]


def _floats_json(a) -> str:
    """float32 values as JSON numbers that read back to the same float32 (9 significant digits), non-finite as the
    strings Newtonsoft writes."""
    a = np.asarray(a, np.float32).reshape(-1)
    if a.size == 0:
        return "[]"
    if np.isfinite(a).all():
        return "[" + ",".join(np.char.mod("%.9g", a.astype(np.float64))) + "]"
    out = []
    for v in a:
        out.append("%.9g" % float(v) if np.isfinite(v) else ('"NaN"' if np.isnan(v) else ('"Infinity"' if v > 0 else '"-Infinity"')))
    return "[" + ",".join(out) + "]"


def _matrix_json(m) -> str:
    m = np.asarray(m, np.float32)
    return "[" + ",".join(_floats_json(row) for row in m) + "]" if m.shape[1] else "[" + ",".join("[]" for _ in range(m.shape[0])) + "]"


def _ffn_json(cfg, W1, b1, W2, b2, extras) -> str:
    d, f = cfg.embedding_dim, cfg.ffn_dim

    def layer(size, input_size, weights, biases, act):
        z = _floats_json(np.zeros(size, np.float32))
        w = _matrix_json(weights if weights is not None else np.zeros((size, 0), np.float32))
        b = _floats_json(biases if biases is not None else np.zeros(size, np.float32))
        return ('{"Size":%d,"InputSize":%d,"Activations":%s,"Biases":%s,"Derivatives":%s,"Deltas":%s,"Weights":%s,"ActivationType":%d}'
                % (size, input_size, z, b, z, z, w, act))

    params = {
        "HuberLossDelta": 1.0, "AccelerationType": ACCEL_CPU, "AccelerationDeviceId": 0,
        "CostFunction": int(extras.get("CostFunction", 0)), "ActivationDistribution": int(extras.get("ActivationDistribution", 0)),
        "L2RegulationLamda": float(extras.get("L2RegulationLamda", 0.0)), "GradientClippingThreshold": float(extras.get("GradientClippingThreshold", 1.0)),
        "GradientExplosionThreshold": 1000.0, "GradientVanishingThreshold": 1e-05,
        "LayerWidths": [d, f, d], "LayerActivations": [0, int(cfg.ffn_activation), 0],
        "inputActivationMin": [0.0] * d, "inputActivationMax": [1.0] * d, "OptimalLearningRate": None, "EpochsTrainedOn": 10,
    }
    return ('{"layers":[' + ",".join([layer(d, 0, None, None, 0), layer(f, d, W1, b1, int(cfg.ffn_activation)), layer(d, f, W2, b2, 0)])
            + '],"parameters":' + json.dumps(params) + "}")


def save_reference_checkpoint(directory, cfg, tensors, params, max_sequence_length, extras=None, adam=None):
    """Writes config.json, weights.bin and ffn/ffn_layer_i.json from the flat arena `params` (a host array as
    b200_lm_download_params returns it).  extras: optional values for the config keys the arena knows nothing about
    (L2RegulationLamda, GradientClippingThreshold, CostFunction, ActivationDistribution, AccelerationDeviceId).
    adam = (first moments, second moments, step index) adds optimizer.bin."""
    extras = dict(extras or {})
    params = np.ascontiguousarray(params, np.float32).reshape(-1)
    d = Path(directory)
    (d / "ffn").mkdir(parents=True, exist_ok=True)
    config = {
        "VocabSize": int(cfg.vocab_size), "MaxSequenceLength": int(max_sequence_length), "EmbeddingDim": int(cfg.embedding_dim),
        "NumHeads": int(cfg.num_heads), "NumLayers": int(cfg.num_layers), "FeedForwardDim": int(cfg.ffn_dim), "UseDecoderOnly": bool(cfg.causal),
        "FFNActivationType": int(cfg.ffn_activation), "AccelerationType": ACCEL_CPU, "AccelerationDeviceId": int(extras.get("AccelerationDeviceId", 0)),
        "L2RegulationLamda": float(extras.get("L2RegulationLamda", 0.0)), "GradientClippingThreshold": float(extras.get("GradientClippingThreshold", 1.0)),
        "DataType": _data_type(cfg), "InputFeatureDim": int(cfg.input_feature_dim), "OutputDim": int(cfg.output_dim if not cfg.discrete else extras.get("OutputDim", 0)),
        "CostFunction": int(extras.get("CostFunction", 0)), "ActivationDistribution": int(extras.get("ActivationDistribution", 0)),
    }
    (d / "config.json").write_text(json.dumps(config, indent=2))
    first, layers, last = _layer_tensor_slices(cfg, tensors)

    def mat(f, t):
        off, r, c = t
        f.write(struct.pack("<ii", r, c))
        f.write(params[off:off + r * c].astype("<f4").tobytes())

    def vec(f, t):
        off, r, c = t
        f.write(struct.pack("<i", r * c))
        f.write(params[off:off + r * c].astype("<f4").tobytes())

    with open(d / "weights.bin", "wb") as f:
        f.write(struct.pack("<?", bool(cfg.discrete)))
        mat(f, first[0])
        if not cfg.discrete:
            vec(f, first[1])
        for lt in layers:
            for t in lt[0:4]:
                mat(f, t)
            for t in lt[4:12]:
                vec(f, t)
        mat(f, last[0])
        vec(f, last[1])
    for i, lt in enumerate(layers):
        get = lambda t: params[t[0]:t[0] + t[1] * t[2]].reshape(t[1], t[2])
        W1, b1, W2, b2 = get(lt[12]), get(lt[13]).reshape(-1), get(lt[14]), get(lt[15]).reshape(-1)
        path = d / "ffn" / f"ffn_layer_{i}.json"
        if path.exists():
            path.unlink()  # "overwrite always (avoid stale files)", LanguageModel.cs:679-681
        path.write_text(_ffn_json(cfg, W1, b1, W2, b2, extras), encoding="utf-8")
    if adam is not None:
        m, v, step = adam
        with open(d / "optimizer.bin", "wb") as f:
            f.write(OPT_MAGIC + struct.pack("<qq", int(step), params.size))
            f.write(np.ascontiguousarray(m, "<f4").tobytes())
            f.write(np.ascontiguousarray(v, "<f4").tobytes())
    elif (d / "optimizer.bin").exists():
        (d / "optimizer.bin").unlink()


def _read_matrix_into(f, dst, rows, cols, what):
    r, c = struct.unpack("<ii", f.read(8))
    if (r, c) != (rows, cols):  # ReadMatrixInto's shape check
        raise ValueError(f"{what}: file holds a {r}x{c} matrix, the model expects {rows}x{cols}")
    dst[:] = np.frombuffer(f.read(4 * r * c), "<f4")


def _read_vector_into(f, dst, n, what):
    (k,) = struct.unpack("<i", f.read(4))
    if k != n:
        raise ValueError(f"{what}: file holds a vector of {k}, the model expects {n}")
    dst[:] = np.frombuffer(f.read(4 * k), "<f4")


def load_reference_checkpoint(directory, make_config, tensor_table):
    """Reads a directory written by LanguageModel.Save (or by save_reference_checkpoint).

    make_config(**kw) builds the library's model configuration; tensor_table(cfg) returns (tensors, total).  Returns
    (cfg, params, config_dict, adam) with adam = (m, v, step) or None."""
    d = Path(directory)
    conf = json.loads((d / "config.json").read_text())
    data_type = int(conf["DataType"])
    discrete = data_type in (DATA_TEXT, DATA_SYMBOLIC)
    with open(d / "weights.bin", "rb") as f:
        (saved_discrete,) = struct.unpack("<?", f.read(1))
        if saved_discrete != discrete:
            raise ValueError("weights.bin and config.json disagree on UsesDiscreteTokens")
        out_dim = int(conf["VocabSize"]) if discrete else int(conf["OutputDim"])
        cfg = make_config(vocab_size=int(conf["VocabSize"]) if discrete else 0, input_feature_dim=0 if discrete else int(conf["InputFeatureDim"]),
                          output_dim=out_dim, embedding_dim=int(conf["EmbeddingDim"]), num_heads=int(conf["NumHeads"]), num_layers=int(conf["NumLayers"]),
                          ffn_dim=int(conf["FeedForwardDim"]), ffn_activation=int(conf["FFNActivationType"]), discrete=discrete,
                          loss="mse" if data_type == DATA_TS_REGRESSION else "ce", causal=bool(conf["UseDecoderOnly"]))
        tensors, total = tensor_table(cfg)
        params = np.zeros(total, np.float32)
        first, layers, last = _layer_tensor_slices(cfg, tensors)
        view = lambda t: params[t[0]:t[0] + t[1] * t[2]]
        _read_matrix_into(f, view(first[0]), first[0][1], first[0][2], "TokenEmbedding" if discrete else "InputProjection")
        if not discrete:
            _read_vector_into(f, view(first[1]), first[1][1] * first[1][2], "InputProjectionBias")
        names = ["WQ", "WK", "WV", "WO", "BiasQ", "BiasK", "BiasV", "BiasO", "LN1Gamma", "LN1Beta", "LN2Gamma", "LN2Beta"]
        for l, lt in enumerate(layers):
            for k in range(4):
                _read_matrix_into(f, view(lt[k]), lt[k][1], lt[k][2], f"layer {l} {names[k]}")
            for k in range(4, 12):
                _read_vector_into(f, view(lt[k]), lt[k][1] * lt[k][2], f"layer {l} {names[k]}")
        _read_matrix_into(f, view(last[0]), last[0][1], last[0][2], "OutputProjection")
        _read_vector_into(f, view(last[1]), last[1][1] * last[1][2], "OutputBias")
        if f.read(1):
            raise ValueError("weights.bin holds more data than the configuration describes")
    for l, lt in enumerate(layers):
        path = d / "ffn" / f"ffn_layer_{l}.json"
        if not path.exists():
            raise FileNotFoundError(f"Missing FFN file: {path}")  # LanguageModel.cs:690-691
        net = json.loads(path.read_text(encoding="utf-8-sig"))
        ls = net["layers"]
        if len(ls) != 3:
            raise ValueError(f"{path}: a transformer block's feed-forward network has three layers, found {len(ls)}")
        for k, (tw, tb) in ((1, (lt[12], lt[13])), (2, (lt[14], lt[15]))):
            W = np.asarray(ls[k]["Weights"], np.float32)
            if W.shape != (tw[1], tw[2]):
                raise ValueError(f"{path}: layer {k} weights are {W.shape}, the model expects {(tw[1], tw[2])}")
            view(tw)[:] = W.reshape(-1)
            view(tb)[:] = np.asarray([float(x) for x in ls[k]["Biases"]], np.float32)
    adam = None
    if (d / "optimizer.bin").exists():
        with open(d / "optimizer.bin", "rb") as f:
            if f.read(8) != OPT_MAGIC:
                raise ValueError("optimizer.bin: bad magic")
            step, n = struct.unpack("<qq", f.read(16))
            if n != total:
                raise ValueError(f"optimizer.bin holds {n} values per moment, the model has {total} parameters")
            m = np.frombuffer(f.read(4 * n), "<f4").copy()
            v = np.frombuffer(f.read(4 * n), "<f4").copy()
            adam = (m, v, int(step))
    return cfg, params, conf, adam
