"""Resident trainers over the C ABI: the hooks TransformerTrainer.TrainBatchDiscrete/Continuous and
NeuralNetwork.TrainBatch route to when the B200 back end is selected, plus the one-process-per-GPU data-parallel
wrapper (torch.distributed / NCCL supplies the collective; every kernel is the library's own).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib as L
from .manager import CudaB200AccelerationManager, _f, _i, _pf, _pi


def make_config(vocab_size=0, input_feature_dim=0, output_dim=None, embedding_dim=64, num_heads=4, num_layers=2, ffn_dim=128,
                ffn_activation="Relu", discrete=True, loss="ce", causal=True, align_floats=64) -> L.LMConfig:
    """TransformerConfig fields that shape the trained tensors (Transformers/MultiTypeTransformer/TransformerConfig.cs)."""
    c = L.LMConfig()
    c.vocab_size, c.input_feature_dim = int(vocab_size), int(input_feature_dim)
    c.output_dim = int(vocab_size if (discrete and output_dim is None) else output_dim)
    c.embedding_dim, c.num_heads, c.num_layers, c.ffn_dim = int(embedding_dim), int(num_heads), int(num_layers), int(ffn_dim)
    c.ffn_activation = L.ACT[ffn_activation] if isinstance(ffn_activation, str) else int(ffn_activation)
    c.discrete = 1 if discrete else 0
    c.loss_kind = 0 if loss == "ce" else 1
    c.causal = 1 if causal else 0
    c.align_floats = int(align_floats)
    return c


class B200LanguageModelTrainer:
    """Device-resident state of one TransformerTrainer (model weights, gradients, activation caches)."""

    def __init__(self, manager: CudaB200AccelerationManager, config: L.LMConfig, max_rows_per_pass: int, params_ptr: int = 0, grads_ptr: int = 0):
        self.mgr, self.lib, self.cfg = manager, manager.lib, config
        n = self.lib.b200_lm_param_count(C.byref(config))
        if n < 0:
            raise ValueError("invalid model configuration")
        self.param_count = int(n)
        h = C.c_void_p()
        manager._ck(self.lib.b200_lm_create(manager.ctx, C.byref(config), C.c_void_p(params_ptr or 0), C.c_void_p(grads_ptr or 0),
                                            int(max_rows_per_pass), C.byref(h)))
        self.h = h
        self._cb = None
        self._optimizer = "sgd"
        self.max_rows_per_pass = int(max_rows_per_pass)
        manager._children.add(self)

    def close(self):
        if getattr(self, "h", None):
            self.lib.b200_lm_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def tensors(self):
        """[(offset, rows, cols)] of every tensor of the flat arena, in weights.bin order with each block's FFN appended."""
        return self._tensors_of(self.cfg)

    def upload_params(self, flat, offset=0):
        a = _f(flat).reshape(-1)
        self.mgr._ck(self.lib.b200_lm_upload_params(self.h, _pf(a), offset, a.size))

    def download_params(self, offset=0, count=None):
        count = self.param_count - offset if count is None else count
        out = np.zeros(count, np.float32)
        self.mgr._ck(self.lib.b200_lm_download_params(self.h, _pf(out), offset, count))
        return out

    def download_grads(self, offset=0, count=None):
        count = self.param_count - offset if count is None else count
        out = np.zeros(count, np.float32)
        self.mgr._ck(self.lib.b200_lm_download_grads(self.h, _pf(out), offset, count))
        return out

    def set_optimizer(self, kind="sgd", beta1=0.9, beta2=0.999, eps=1e-8):
        if kind not in ("sgd", "adam"):
            raise ValueError("optimizer must be 'sgd' or 'adam'")
        self.mgr._ck(self.lib.b200_lm_set_optimizer(self.h, L.OPT_ADAM if kind == "adam" else L.OPT_SGD, beta1, beta2, eps))
        self._optimizer = kind

    def set_grad_ready_callback(self, fn):
        """fn(offset, count, cuda_event_ptr) or None."""
        if fn is None:
            self._cb = L.GRAD_READY_FN(0)
        else:
            self._cb = L.GRAD_READY_FN(lambda user, off, cnt, ev: fn(int(off), int(cnt), int(ev or 0)))
        self.mgr._ck(self.lib.b200_lm_set_grad_ready_callback(self.h, self._cb, None))

    # ---- TransformerTrainer.TrainBatchDiscrete / TrainBatchContinuous
    def train_step_discrete(self, tokens, seq_offsets, lr, use_clip=True, clip_threshold=1.0, do_step=True):
        t, o = _i(tokens), _i(seq_offsets)
        loss, norm, valid = C.c_float(0), C.c_float(0), C.c_int32(0)
        self.mgr._ck(self.lib.b200_lm_train_step_discrete(self.h, _pi(t), _pi(o), len(o) - 1, lr, int(bool(use_clip)), clip_threshold, int(bool(do_step)),
                                                          C.byref(loss), C.byref(norm), C.byref(valid)))
        return loss.value, norm.value, valid.value

    def train_step_continuous(self, features, seq_offsets, reg_targets=None, class_targets=None, lr=1e-3, use_clip=True, clip_threshold=1.0, do_step=True):
        x, o = _f(features), _i(seq_offsets)
        r = None if reg_targets is None else _f(reg_targets)
        k = None if class_targets is None else _i(class_targets)
        loss, norm, valid = C.c_float(0), C.c_float(0), C.c_int32(0)
        self.mgr._ck(self.lib.b200_lm_train_step_continuous(self.h, _pf(x), _pf(r), None if k is None else _pi(k), _pi(o), len(o) - 1, lr, int(bool(use_clip)),
                                                            clip_threshold, int(bool(do_step)), C.byref(loss), C.byref(norm), C.byref(valid)))
        return loss.value, norm.value, valid.value

    # ---- TransformerTrainer.Validate / ValidateContinuous: forward + loss only
    def validate_discrete(self, tokens, seq_offsets):
        """(token-weighted mean cross-entropy, contributing rows) of the valid sequences."""
        t, o = _i(tokens), _i(seq_offsets)
        loss, items = C.c_float(0), C.c_int32(0)
        self.mgr._ck(self.lib.b200_lm_validate_discrete(self.h, _pi(t), _pi(o), len(o) - 1, C.byref(loss), C.byref(items)))
        return loss.value, items.value

    def validate_continuous(self, features, seq_offsets, reg_targets=None, class_targets=None):
        x, o = _f(features), _i(seq_offsets)
        r = None if reg_targets is None else _f(reg_targets)
        k = None if class_targets is None else _i(class_targets)
        loss, items = C.c_float(0), C.c_int32(0)
        self.mgr._ck(self.lib.b200_lm_validate_continuous(self.h, _pf(x), _pf(r), None if k is None else _pi(k), _pi(o), len(o) - 1,
                                                          C.byref(loss), C.byref(items)))
        return loss.value, items.value

    # ---- optimiser state (checkpoints that resume on the device)
    def download_optimizer_state(self):
        """(first moments, second moments, step index) of Adam, in the layout of the parameter arena."""
        m, v = np.zeros(self.param_count, np.float32), np.zeros(self.param_count, np.float32)
        self.mgr._ck(self.lib.b200_lm_download_optimizer_state(self.h, 0, _pf(m), 0, m.size))
        self.mgr._ck(self.lib.b200_lm_download_optimizer_state(self.h, 1, _pf(v), 0, v.size))
        step = C.c_int32(0)
        self.mgr._ck(self.lib.b200_lm_get_step_index(self.h, C.byref(step)))
        return m, v, step.value

    def upload_optimizer_state(self, m, v, step_index):
        m, v = _f(m).reshape(-1), _f(v).reshape(-1)
        self.mgr._ck(self.lib.b200_lm_upload_optimizer_state(self.h, 0, _pf(m), 0, m.size))
        self.mgr._ck(self.lib.b200_lm_upload_optimizer_state(self.h, 1, _pf(v), 0, v.size))
        self.mgr._ck(self.lib.b200_lm_set_step_index(self.h, int(step_index)))

    def save_checkpoint(self, directory, max_sequence_length=None, extras=None):
        """LanguageModel.Save (LanguageModel.cs:706-765): config.json, weights.bin and ffn/ffn_layer_i.json in the
        reference's own format, straight from the device arena, so that LanguageModel.Load opens the result.  With Adam
        selected the moments and the step index go into optimizer.bin beside them (the reference's SGD keeps no state)."""
        from .checkpoint import save_reference_checkpoint

        adam = self.download_optimizer_state() if self._optimizer == "adam" else None
        save_reference_checkpoint(directory, self.cfg, self.tensors(), self.download_params(), max_sequence_length or self.max_rows_per_pass + 1,
                                  extras, adam)

    def load_checkpoint(self, directory):
        """LanguageModel.Load (LanguageModel.cs:769-839) into this trainer: the directory may come from the reference or
        from save_checkpoint.  The stored shape must be this trainer's.  Returns config.json as a dict."""
        from .checkpoint import load_reference_checkpoint

        cfg, params, conf, adam = load_reference_checkpoint(directory, make_config, lambda c: (self._tensors_of(c), int(self.lib.b200_lm_param_count(C.byref(c)))))
        mine = [getattr(self.cfg, n) for n, _ in L.LMConfig._fields_ if n != "align_floats"]
        theirs = [getattr(cfg, n) for n, _ in L.LMConfig._fields_ if n != "align_floats"]
        if mine != theirs:
            raise ValueError(f"checkpoint shape {theirs} does not match this trainer's {mine}")
        if cfg.align_floats != self.cfg.align_floats:  # re-lay the tensors out in this trainer's arena
            flat = np.zeros(self.param_count, np.float32)
            for (so, r, c), (do, _, _) in zip(self._tensors_of(cfg), self.tensors()):
                flat[do:do + r * c] = params[so:so + r * c]
            params = flat
        self.upload_params(params)
        if adam is not None:
            if self._optimizer != "adam":
                raise ValueError("the checkpoint holds Adam state but this trainer's optimizer is SGD: call set_optimizer('adam') first")
            m, v, step = adam
            if cfg.align_floats != self.cfg.align_floats:
                raise ValueError("optimizer.bin was written with another arena alignment")
            self.upload_optimizer_state(m, v, step)
        return conf

    def _tensors_of(self, cfg):
        out = []
        for i in range(self.lib.b200_lm_tensor_count(C.byref(cfg))):
            off, r, c = C.c_int64(), C.c_int32(), C.c_int32()
            self.lib.b200_lm_tensor_info(C.byref(cfg), i, C.byref(off), C.byref(r), C.byref(c))
            out.append((off.value, r.value, c.value))
        return out

    # ---- LanguageModel.Generate (decoder path): incremental decoding with a device key/value cache
    def generator(self, max_len):
        return B200Generator(self, max_len)

    # ---- device-resident batches
    def prepare_discrete(self, tokens, seq_offsets):
        """Plan, pack and copy a batch to the device once; returns a handle for train_step_batch / accumulate_batch."""
        t, o = _i(tokens), _i(seq_offsets)
        h = C.c_void_p()
        self.mgr._ck(self.lib.b200_lm_batch_create_discrete(self.h, _pi(t), _pi(o), len(o) - 1, C.byref(h)))
        return h

    def prepare_continuous(self, features, seq_offsets, reg_targets=None, class_targets=None):
        x, o = _f(features), _i(seq_offsets)
        r = None if reg_targets is None else _f(reg_targets)
        k = None if class_targets is None else _i(class_targets)
        h = C.c_void_p()
        self.mgr._ck(self.lib.b200_lm_batch_create_continuous(self.h, _pf(x), _pf(r), None if k is None else _pi(k), _pi(o), len(o) - 1, C.byref(h)))
        return h

    def release_batch(self, batch):
        self.lib.b200_lm_batch_destroy(batch)

    def train_step_batch(self, batch, lr, use_clip=True, clip_threshold=1.0, do_step=True):
        loss, norm, valid = C.c_float(0), C.c_float(0), C.c_int32(0)
        self.mgr._ck(self.lib.b200_lm_train_step_batch(self.h, batch, lr, int(bool(use_clip)), clip_threshold, int(bool(do_step)),
                                                       C.byref(loss), C.byref(norm), C.byref(valid)))
        return loss.value, norm.value, valid.value

    def accumulate_batch(self, batch):
        ls, vc = C.c_float(0), C.c_int32(0)
        self.mgr._ck(self.lib.b200_lm_accumulate_batch(self.h, batch, C.byref(ls), C.byref(vc)))
        return ls.value, vc.value

    # ---- data-parallel decomposition
    def zero_grads(self):
        self.mgr._ck(self.lib.b200_lm_zero_grads(self.h))

    def accumulate_discrete(self, tokens, seq_offsets):
        t, o = _i(tokens), _i(seq_offsets)
        ls, vc = C.c_float(0), C.c_int32(0)
        self.mgr._ck(self.lib.b200_lm_accumulate_discrete(self.h, _pi(t), _pi(o), len(o) - 1, C.byref(ls), C.byref(vc)))
        return ls.value, vc.value

    def accumulate_continuous(self, features, seq_offsets, reg_targets=None, class_targets=None):
        x, o = _f(features), _i(seq_offsets)
        r = None if reg_targets is None else _f(reg_targets)
        k = None if class_targets is None else _i(class_targets)
        ls, vc = C.c_float(0), C.c_int32(0)
        self.mgr._ck(self.lib.b200_lm_accumulate_continuous(self.h, _pf(x), _pf(r), None if k is None else _pi(k), _pi(o), len(o) - 1, C.byref(ls), C.byref(vc)))
        return ls.value, vc.value

    def apply_step(self, global_valid_count, lr, use_clip=True, clip_threshold=1.0, do_step=True):
        norm = C.c_float(0)
        self.mgr._ck(self.lib.b200_lm_apply_step(self.h, int(global_valid_count), lr, int(bool(use_clip)), clip_threshold, int(bool(do_step)), C.byref(norm)))
        return norm.value

    def timings_ms(self):
        out = (C.c_float * 4)()
        self.lib.b200_lm_get_timings(self.h, out)
        return {"forward": out[0], "loss": out[1], "backward": out[2], "step": out[3]}


class B200Generator:
    """One decoding session: `step(token)` returns the next-token logits after pushing the token through the model at
    the next position (the caller samples, as LanguageModel.Generate does with its own random generator); `greedy`
    continues a prompt with arg-max choices entirely on the device."""

    def __init__(self, trainer, max_len):
        self.t, self.lib, self.mgr = trainer, trainer.lib, trainer.mgr
        self.h = C.c_void_p()
        self.mgr._ck(self.lib.b200_lm_gen_create(trainer.h, int(max_len), C.byref(self.h)))
        self.max_len = int(max_len)
        self.out_dim = int(trainer.cfg.output_dim)

    def reset(self):
        self.mgr._ck(self.lib.b200_lm_gen_reset(self.h))

    def __len__(self):
        n = C.c_int32(0)
        self.mgr._ck(self.lib.b200_lm_gen_length(self.h, C.byref(n)))
        return n.value

    def single_kernel(self) -> bool:
        """True when each token runs as one cooperative kernel (the preferred path)."""
        return bool(self.lib.b200_lm_gen_single_kernel(self.h))

    def set_single_kernel(self, on: bool):
        """False selects the separate-launch path (CUDA graph from the second token on) on purpose."""
        self.mgr._ck(self.lib.b200_lm_gen_set_single_kernel(self.h, int(bool(on))))

    def graph_nodes(self):
        """Kernel launches replayed per token from the captured CUDA graph (0 while the session still issues plain launches)."""
        n = C.c_int32(0)
        self.mgr._ck(self.lib.b200_lm_gen_graph_nodes(self.h, C.byref(n)))
        return n.value

    def step(self, token_id):
        out = np.zeros(self.out_dim, np.float32)
        self.mgr._ck(self.lib.b200_lm_gen_step(self.h, int(token_id), _pf(out)))
        return out

    def greedy(self, prompt, max_new):
        p = _i(prompt)
        out = np.zeros(len(p) + int(max_new), np.int32)
        n = C.c_int32(0)
        self.mgr._ck(self.lib.b200_lm_gen_greedy(self.h, _pi(p), len(p), int(max_new), _pi(out), C.byref(n)))
        return out[:n.value]

    def close(self):
        if getattr(self, "h", None):
            self.lib.b200_lm_gen_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class B200MlpBatchTrainer:
    """NeuralNetwork.TrainBatch state on the device (the role AccelerationGPUBatch plays in the reference)."""

    def __init__(self, manager: CudaB200AccelerationManager, widths, activations, cost="mse", huber_delta=1.0, l2_lambda=0.0,
                 clip_threshold=1.0, max_batch=256):
        self.mgr, self.lib = manager, manager.lib
        self.widths = [int(w) for w in widths]
        wd = np.asarray(self.widths, np.int32)
        ac = np.asarray([L.ACT[a] if isinstance(a, str) else int(a) for a in activations], np.int32)
        h = C.c_void_p()
        manager._ck(self.lib.b200_mlp_create(manager.ctx, len(self.widths), _pi(wd), _pi(ac), L.COST[cost] if isinstance(cost, str) else int(cost),
                                             huber_delta, l2_lambda, clip_threshold, int(max_batch), C.byref(h)))
        self.h = h
        manager._children.add(self)

    def close(self):
        if getattr(self, "h", None):
            self.lib.b200_mlp_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def upload_layer(self, layer, weights, biases):
        w, b = _f(weights), _f(biases)
        if w.shape != (self.widths[layer], self.widths[layer - 1]) or b.shape != (self.widths[layer],):
            raise ValueError("layer shape mismatch")
        self.mgr._ck(self.lib.b200_mlp_upload_layer(self.h, layer, _pf(w), _pf(b)))

    def download_layer(self, layer):
        w = np.zeros((self.widths[layer], self.widths[layer - 1]), np.float32)
        b = np.zeros(self.widths[layer], np.float32)
        self.mgr._ck(self.lib.b200_mlp_download_layer(self.h, layer, _pf(w), _pf(b)))
        return w, b

    def learn_batch(self, X, Y, lr, in_min=None, in_max=None):
        x, y = _f(X), _f(Y)
        mn = None if in_min is None else _f(in_min)
        mx = None if in_max is None else _f(in_max)
        norm = C.c_float(0)
        self.mgr._ck(self.lib.b200_mlp_learn_batch(self.h, _pf(x), _pf(y), x.shape[0], lr, _pf(mn), _pf(mx), C.byref(norm)))
        return norm.value


def split_sequences(n_seq: int, rank: int, world: int):
    """Contiguous shard of sequence indices for this rank (the batch is split by sequence): b200_dp_shard."""
    lo, hi = C.c_int32(), C.c_int32()
    if L.load().b200_dp_shard(int(n_seq), int(rank), int(world), C.byref(lo), C.byref(hi)) != L.OK:
        raise ValueError(f"rank {rank} outside a world of {world}")
    return lo.value, hi.value


def _bundled_nccl():
    """Path of the NCCL build that ships with the installed torch wheel, if any (one NCCL per process is the aim)."""
    try:
        import nvidia.nccl as pkg
        from pathlib import Path

        for base in list(getattr(pkg, "__path__", [])):
            cand = Path(base) / "lib" / "libnccl.so.2"
            if cand.exists():
                return str(cand)
    except Exception:
        pass
    return None


class DataParallelLMTrainer:
    """One process per GPU; a thin caller of the library's data-parallel entry points (b200_dp_*).

    Every rank holds the full model; the batch is split by sequence; gradients are summed with bucketed NCCL all-reduces
    that the LIBRARY issues on its own communication stream as soon as each range of the gradient arena is final
    (output projection first, then the blocks last to first, then the embedding), overlapping the remaining backward;
    loss sum, valid count and a failure flag travel in one small all-reduce; every rank then applies the identical fused
    clip-and-step kernel to identical data.  torch.distributed is only the rendezvous here: it tells the ranks apart and
    carries the 128-byte communicator id from rank 0 to the others."""

    def __init__(self, config: L.LMConfig, max_rows_per_pass: int, device_index: int, process_group=None, gemm_mode=L.GEMM_AUTO):
        import torch
        import torch.distributed as dist

        self.torch, self.dist, self.pg = torch, dist, process_group
        self.rank, self.world = dist.get_rank(process_group), dist.get_world_size(process_group)
        self.device = torch.device("cuda", device_index)
        torch.cuda.set_device(self.device)
        self.mgr = CudaB200AccelerationManager(device_index, gemm_mode)
        self.compute = torch.cuda.Stream(device=self.device)  # torch-visible, so that callers can time it with torch events
        self.mgr.set_stream(self.compute.cuda_stream)
        self.lm = B200LanguageModelTrainer(self.mgr, config, max_rows_per_pass)
        self.dp = None
        if self.world > 1:
            lib = self.mgr.lib
            path = _bundled_nccl()
            if path:
                lib.b200_dp_set_nccl_library(path.encode())  # ignored once a copy is loaded
            ident = (C.c_uint8 * 128)()
            if self.rank == 0 and lib.b200_dp_unique_id(ident) != L.OK:
                raise L.B200Error("NCCL could not be loaded or refused to create a communicator id")
            box = [bytes(ident)]
            dist.broadcast_object_list(box, src=dist.get_global_rank(process_group, 0) if process_group is not None else 0, group=process_group)
            ident = (C.c_uint8 * 128).from_buffer_copy(box[0])
            h = C.c_void_p()
            self.mgr._ck(lib.b200_dp_create_rank(self.lm.h, ident, self.rank, self.world, C.byref(h)))
            self.dp = h

    def close(self):
        """Release the device state now, communicator first."""
        if getattr(self, "lm", None) is not None:
            self.torch.cuda.synchronize(self.device)
            if self.dp is not None:
                self.mgr.lib.b200_dp_destroy(self.dp)
                self.dp = None
            self.lm.close()
            self.mgr.Dispose()
            self.lm = None

    def set_deadline_ms(self, ms: int):
        if self.dp is not None:
            self.mgr._ck(self.mgr.lib.b200_dp_set_deadline_ms(self.dp, int(ms)))

    def broadcast_params(self, flat_host=None):
        """Rank 0 uploads flat_host (when given); every rank then receives rank 0's parameter arena."""
        if flat_host is not None and self.rank == 0:
            self.lm.upload_params(flat_host)
        if self.dp is not None:
            self.mgr._ck(self.mgr.lib.b200_dp_broadcast_params(self.dp, 0))
        elif flat_host is not None and self.rank != 0:
            self.lm.upload_params(flat_host)

    def prepare_discrete(self, tokens, seq_offsets):
        """Copy this rank's shard of the GLOBAL batch to the device once; returns a handle for train_step_prepared."""
        if self.dp is None:
            return self.lm.prepare_discrete(tokens, seq_offsets)
        t, o = _i(tokens), _i(seq_offsets)
        if t.size == 0:
            t = np.zeros(1, np.int32)
        h = C.c_void_p()
        self.mgr._ck(self.mgr.lib.b200_dp_batch_create_discrete(self.dp, _pi(t), _pi(o), len(o) - 1, C.byref(h)))
        return h

    def prepare_continuous(self, features, seq_offsets, reg_targets=None, class_targets=None):
        if self.dp is None:
            return self.lm.prepare_continuous(features, seq_offsets, reg_targets, class_targets)
        x, o = _f(features), _i(seq_offsets)
        r = None if reg_targets is None else _f(reg_targets)
        k = None if class_targets is None else _i(class_targets)
        h = C.c_void_p()
        self.mgr._ck(self.mgr.lib.b200_dp_batch_create_continuous(self.dp, _pf(x), _pf(r), None if k is None else _pi(k), _pi(o), len(o) - 1, C.byref(h)))
        return h

    def train_step_continuous(self, features, seq_offsets, reg_targets=None, class_targets=None, lr=1e-3, use_clip=True, clip_threshold=1.0, do_step=True):
        """features / targets / seq_offsets describe the GLOBAL batch in host memory; this rank trains its shard."""
        if self.dp is None:
            return self.lm.train_step_continuous(features, seq_offsets, reg_targets, class_targets, lr, use_clip, clip_threshold, do_step)
        x, o = _f(features), _i(seq_offsets)
        r = None if reg_targets is None else _f(reg_targets)
        k = None if class_targets is None else _i(class_targets)
        loss, norm, valid = C.c_float(0), C.c_float(0), C.c_int32(0)
        self.mgr._ck(self.mgr.lib.b200_dp_train_step_continuous(self.dp, _pf(x), _pf(r), None if k is None else _pi(k), _pi(o), len(o) - 1, lr,
                                                                int(bool(use_clip)), clip_threshold, int(bool(do_step)), C.byref(loss), C.byref(norm),
                                                                C.byref(valid)))
        return loss.value, norm.value, valid.value

    def train_step_prepared(self, batch, lr, use_clip=True, clip_threshold=1.0, do_step=True):
        if self.dp is None:
            return self.lm.train_step_batch(batch, lr, use_clip, clip_threshold, do_step)
        loss, norm, valid = C.c_float(0), C.c_float(0), C.c_int32(0)
        self.mgr._ck(self.mgr.lib.b200_dp_train_step_batch(self.dp, batch, lr, int(bool(use_clip)), clip_threshold, int(bool(do_step)),
                                                           C.byref(loss), C.byref(norm), C.byref(valid)))
        return loss.value, norm.value, valid.value

    def train_step_discrete(self, tokens, seq_offsets, lr, use_clip=True, clip_threshold=1.0, do_step=True):
        """tokens/seq_offsets describe the GLOBAL batch in host memory; this rank trains its shard."""
        if self.dp is None:
            return self.lm.train_step_discrete(tokens, seq_offsets, lr, use_clip, clip_threshold, do_step)
        t, o = _i(tokens), _i(seq_offsets)
        if t.size == 0:
            t = np.zeros(1, np.int32)
        loss, norm, valid = C.c_float(0), C.c_float(0), C.c_int32(0)
        self.mgr._ck(self.mgr.lib.b200_dp_train_step_discrete(self.dp, _pi(t), _pi(o), len(o) - 1, lr, int(bool(use_clip)), clip_threshold,
                                                              int(bool(do_step)), C.byref(loss), C.byref(norm), C.byref(valid)))
        return loss.value, norm.value, valid.value

    def timings_ms(self):
        """Phase times of the last step on the device, with the communication the step had to wait for."""
        out = self.lm.timings_ms()
        if self.dp is not None:
            ms = (C.c_float * 2)()
            self.mgr.lib.b200_dp_get_timings(self.dp, ms)
            out["comm_exposed"], out["comm_span"] = ms[0], ms[1]
        else:
            out["comm_exposed"], out["comm_span"] = 0.0, 0.0
        return out


class B200DataParallelGroup:
    """All GPUs of one process behind one handle (b200_dp_group_*): what a single-process host such as the reference's
    C# trainer calls.  One context, one trainer and one rank per listed device, driven by one host thread each."""

    def __init__(self, devices, config: L.LMConfig, max_rows_per_pass: int, gemm_mode=L.GEMM_AUTO):
        self.lib = L.load()
        path = _bundled_nccl()
        if path:
            self.lib.b200_dp_set_nccl_library(path.encode())
        dev = np.asarray(list(devices), np.int32)
        h = C.c_void_p()
        rc = self.lib.b200_dp_group_create(_pi(dev), len(dev), C.byref(config), int(max_rows_per_pass), int(gemm_mode), C.byref(h))
        if rc != L.OK:
            raise L.B200Error(f"b200_dp_group_create failed with status {rc}")
        self.h, self.cfg, self.n = h, config, len(dev)
        self.param_count = int(self.lib.b200_lm_param_count(C.byref(config)))

    def _ck(self, rc):
        if rc != L.OK:
            msg = self.lib.b200_dp_group_last_error(self.h).decode("utf-8", "replace")
            if rc == L.ERR_OUT_OF_RANGE:
                raise IndexError(msg)
            if rc in (L.ERR_INVALID_ARG, L.ERR_SHAPE):
                raise ValueError(msg)
            raise L.B200Error(f"status {rc}: {msg}")

    def close(self):
        if getattr(self, "h", None):
            self.lib.b200_dp_group_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_optimizer(self, kind="sgd", beta1=0.9, beta2=0.999, eps=1e-8):
        self._ck(self.lib.b200_dp_group_set_optimizer(self.h, L.OPT_ADAM if kind == "adam" else L.OPT_SGD, beta1, beta2, eps))

    def upload_params(self, flat):
        a = _f(flat).reshape(-1)
        self._ck(self.lib.b200_dp_group_upload_params(self.h, _pf(a), 0, a.size))

    def download_params(self, rank=0):
        out = np.zeros(self.param_count, np.float32)
        rc = self.lib.b200_lm_download_params(C.c_void_p(self.lib.b200_dp_group_trainer(self.h, rank)), _pf(out), 0, out.size)
        self._ck(rc)
        return out

    def download_grads(self, rank=0):
        out = np.zeros(self.param_count, np.float32)
        self._ck(self.lib.b200_lm_download_grads(C.c_void_p(self.lib.b200_dp_group_trainer(self.h, rank)), _pf(out), 0, out.size))
        return out

    def train_step_discrete(self, tokens, seq_offsets, lr, use_clip=True, clip_threshold=1.0, do_step=True):
        t, o = _i(tokens), _i(seq_offsets)
        if t.size == 0:
            t = np.zeros(1, np.int32)
        loss, norm, valid = C.c_float(0), C.c_float(0), C.c_int32(0)
        self._ck(self.lib.b200_dp_group_train_step_discrete(self.h, _pi(t), _pi(o), len(o) - 1, lr, int(bool(use_clip)), clip_threshold,
                                                           int(bool(do_step)), C.byref(loss), C.byref(norm), C.byref(valid)))
        return loss.value, norm.value, valid.value
