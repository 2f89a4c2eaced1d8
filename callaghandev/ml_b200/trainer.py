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
        out = []
        for i in range(self.lib.b200_lm_tensor_count(C.byref(self.cfg))):
            off, r, c = C.c_int64(), C.c_int32(), C.c_int32()
            self.lib.b200_lm_tensor_info(C.byref(self.cfg), i, C.byref(off), C.byref(r), C.byref(c))
            out.append((off.value, r.value, c.value))
        return out

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
        self.mgr._ck(self.lib.b200_lm_set_optimizer(self.h, L.OPT_ADAM if kind == "adam" else L.OPT_SGD, beta1, beta2, eps))

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

    def save_checkpoint(self, path):
        """Parameters, Adam moments and step index in one .npz (the reference's weights.bin holds the parameters only)."""
        blobs = {"params": self.download_params()}
        try:
            m, v, step = self.download_optimizer_state()
            blobs.update(adam_m=m, adam_v=v, step_index=np.int64(step))
        except Exception:  # SGD keeps no state
            pass
        np.savez(path, **blobs)

    def load_checkpoint(self, path):
        z = np.load(path)
        self.upload_params(z["params"])
        if "adam_m" in z:
            self.upload_optimizer_state(z["adam_m"], z["adam_v"], int(z["step_index"]))

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
    """Contiguous shard of sequence indices for this rank (the batch is split by sequence)."""
    base, rem = divmod(n_seq, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def reduce_host_scalars(dist, loss_sum: float, valid: int, device=None, group=None):
    """Sum (loss_sum, valid_count) over ranks with one small all-reduce."""
    import torch

    t = torch.tensor([float(loss_sum), float(valid)], dtype=torch.float64, device=device if device is not None else "cpu")
    dist.all_reduce(t, group=group)
    return float(t[0].item()), int(round(t[1].item()))


class DataParallelLMTrainer:
    """One process per GPU.  Every rank holds the full model; the batch is split by sequence; gradients are summed with
    bucketed all-reduces issued on a communication stream as soon as each range of the gradient arena is final
    (output projection first, then the blocks last to first, then the embedding), overlapping the remaining backward;
    the loss sum and valid-sequence count travel in one small all-reduce; every rank then applies the identical fused
    clip-and-step kernel to identical data, so no weight broadcast is needed after the first."""

    def __init__(self, config: L.LMConfig, max_rows_per_pass: int, device_index: int, process_group=None, gemm_mode=L.GEMM_AUTO):
        import torch
        import torch.distributed as dist

        self.torch, self.dist, self.pg = torch, dist, process_group
        self.rank, self.world = dist.get_rank(process_group), dist.get_world_size(process_group)
        self.device = torch.device("cuda", device_index)
        torch.cuda.set_device(self.device)
        self.mgr = CudaB200AccelerationManager(device_index, gemm_mode)
        n = int(self.mgr.lib.b200_lm_param_count(C.byref(config)))
        self.params = torch.zeros(n, dtype=torch.float32, device=self.device)
        self.grads = torch.zeros(n, dtype=torch.float32, device=self.device)
        self.compute = torch.cuda.Stream(device=self.device)
        self.comm = torch.cuda.Stream(device=self.device)
        self.mgr.set_stream(self.compute.cuda_stream)
        self.lm = B200LanguageModelTrainer(self.mgr, config, max_rows_per_pass, self.params.data_ptr(), self.grads.data_ptr())
        self._pending = []
        self.lm.set_grad_ready_callback(self._on_ready if self.world > 1 else None)

    def close(self):
        """Release the device state now (the callback holds a reference back to this object, so without this the
        pair is only collected at interpreter exit)."""
        if getattr(self, "lm", None) is not None:
            self.torch.cuda.synchronize(self.device)
            self.lm.set_grad_ready_callback(None)
            self.lm.close()
            self.mgr.Dispose()
            self.lm = None

    def _on_ready(self, offset, count, event_ptr):
        torch = self.torch
        ev = torch.cuda.Event()
        ev.record(self.compute)  # the library recorded its own event on the same stream just before; this one is torch-visible
        self.comm.wait_event(ev)
        with torch.cuda.stream(self.comm):
            self._pending.append(self.dist.all_reduce(self.grads[offset:offset + count], group=self.pg, async_op=True))

    def broadcast_params(self, flat_host=None):
        torch = self.torch
        if flat_host is not None and self.rank == 0:
            self.params.copy_(torch.from_numpy(np.ascontiguousarray(flat_host, dtype=np.float32)))
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            self.dist.broadcast(self.params, src=0, group=self.pg)
        torch.cuda.synchronize(self.device)

    def shard(self, tokens, seq_offsets):
        """This rank's contiguous slice of a GLOBAL batch, as (tokens, offsets) re-based to zero."""
        off = np.asarray(seq_offsets, np.int32)
        lo, hi = split_sequences(len(off) - 1, self.rank, self.world)
        return np.ascontiguousarray(np.asarray(tokens, np.int32)[off[lo]:off[hi]]), (off[lo:hi + 1] - off[lo]).astype(np.int32)

    def prepare_discrete(self, tokens, seq_offsets):
        """Copy this rank's shard of the global batch to the device once; returns a handle for train_step_prepared."""
        t, o = self.shard(tokens, seq_offsets)
        if t.size == 0:
            t = np.zeros(1, np.int32)  # an empty shard is still a batch: it announces every gradient range to its peers
        return self.lm.prepare_discrete(t, o)

    def _finish(self, ls, vc, lr, use_clip, clip_threshold, do_step):
        if self.world > 1:
            with self.torch.cuda.stream(self.compute):  # Work.wait() orders the *current* stream after the collective
                for w in self._pending:
                    w.wait()
            self.compute.wait_stream(self.comm)
            ls, vc = reduce_host_scalars(self.dist, ls, vc, self.device, self.pg)
        norm = self.lm.apply_step(vc, lr, use_clip, clip_threshold, do_step)
        return (ls / vc if vc else 0.0), norm, vc

    def train_step_prepared(self, batch, lr, use_clip=True, clip_threshold=1.0, do_step=True):
        self._pending.clear()
        self.lm.zero_grads()
        ls, vc = self.lm.accumulate_batch(batch)
        return self._finish(ls, vc, lr, use_clip, clip_threshold, do_step)

    def train_step_discrete(self, tokens, seq_offsets, lr, use_clip=True, clip_threshold=1.0, do_step=True):
        """tokens/seq_offsets describe the GLOBAL batch in host memory; this rank trains its shard."""
        t, o = self.shard(tokens, seq_offsets)
        self._pending.clear()
        self.lm.zero_grads()
        if t.size == 0:
            t = np.zeros(1, np.int32)
        # An empty or all-invalid shard still goes through the library: it announces the same gradient ranges in the
        # same order as a rank that trained, so every rank issues identical collectives.
        ls, vc = self.lm.accumulate_discrete(t, o)
        return self._finish(ls, vc, lr, use_clip, clip_threshold, do_step)
