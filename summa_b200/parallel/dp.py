"""Data-parallel group: symmetric (peer-mapped) flat buffers and the fused
reduce-scatter + clip + AdamW + all-gather step.

The reference has no distributed path at all (`summa-llm/src/model/backend.rs:39-55`
always picks one device); this is the B200 design for its single-device
`gradient_norm_and_clip` → optimizer step (`summa-train/src/trainer.rs:1952-1975`).

Two execution modes:
  * `fused` (CUDA): flat gradient / parameter buffers are allocated in symmetric memory
    (one allocation per rank, mapped into every peer's address space over NVLink). The
    step is two kernels from `csrc/comm.cu` that reduce, clip, update and redistribute
    with plain peer loads/stores issued from inside the kernels.
  * `collective` (any backend, including gloo on CPU): `reduce_scatter_tensor` →
    local AdamW → `all_gather_into_tensor`. It is the measured baseline for the fused
    path and the oracle in its tests, and it is what CPU ranks run.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..ops import native


class DataParallelGroup:
    def __init__(self, group, device: torch.device, mode: Optional[str] = None):
        self.group = group
        self.device = device
        self.rank = dist.get_rank(group)
        self.world_size = dist.get_world_size(group)
        if mode is None:
            mode = os.environ.get("SUMMA_DP_MODE", "fused" if device.type == "cuda" else "collective")
        self.mode = mode
        self.epoch = 0
        self._handles: Dict[str, object] = {}
        self._tensors: Dict[str, torch.Tensor] = {}
        self._ptr_arrays: Dict[str, object] = {}
        self._mc_ptrs: Dict[str, int] = {}
        # NVLS (`multimem.ld_reduce` / `multimem.st` through the NVSwitch multicast object of the
        # symmetric buffers) instead of per-peer loads and stores, wherever the allocation has a multicast
        # address: 59.2 ms against 60.6 ms per llama-350m step on 8 GPUs. SUMMA_DP_MULTIMEM=0 turns it off
        # (failure-path tests do: a rank that dies while bound to a multicast object faults its peers).
        self.multimem = os.environ.get("SUMMA_DP_MULTIMEM", "1") == "1"
        if self.mode == "fused":
            import torch.distributed._symmetric_memory as symm_mem
            self._symm = symm_mem
            native.register("sb_dp_sig_words", [])
            sig = self.alloc_symmetric(native.call_value("sb_dp_sig_words"), torch.int32, "sig")
            sig.zero_()
            self._scratch = torch.zeros(8, device=device, dtype=torch.float32)
            self._reduced: Optional[torch.Tensor] = None
            step_sig = ([native.P] * 8 + [native.L, native.L, native.I, native.I, ctypes.c_uint] +
                        [native.F] * 9 + [native.P, native.L, native.P, native.P, native.P])
            native.register("sb_dp_fused_step", step_sig)
            native.register("sb_dp_update_step", step_sig)
            native.register("sb_dp_bucket_reduce",
                            [native.P] * 4 + [native.L] * 4 + [native.I] * 4 + [ctypes.c_uint, native.P, native.I, native.P])
            self._bucket_epoch = None          # epoch of a step whose buckets are being reduced during its backward
            torch.cuda.synchronize()
            dist.barrier(group)

    # ------------------------------------------------------------------ memory
    def alloc_symmetric(self, numel: int, dtype: torch.dtype, name: str) -> torch.Tensor:
        """A flat tensor whose storage every peer can address; returns the local view."""
        if self.mode != "fused":
            t = torch.zeros(numel, device=self.device, dtype=dtype)
            self._tensors[name] = t
            return t
        t = self._symm.empty(numel, dtype=dtype, device=self.device)
        hdl = self._symm.rendezvous(t, self.group.group_name)
        t.zero_()
        self._handles[name] = hdl
        self._tensors[name] = t
        ptrs = [int(p) for p in hdl.buffer_ptrs]
        self._ptr_arrays[name] = (ctypes.c_void_p * self.world_size)(*ptrs)
        self._mc_ptrs[name] = int(getattr(hdl, "multicast_ptr", 0) or 0)
        return t

    def peer_ptrs(self, name: str):
        return self._ptr_arrays[name]

    def barrier(self) -> None:
        if self.device.type == "cuda":
            torch.cuda.synchronize()
        dist.barrier(self.group)

    # ------------------------------------------------------------------ step
    def all_reduce(self, t: torch.Tensor) -> None:
        dist.all_reduce(t, group=self.group)

    def fused_step(self, engine, lr: float, bc1: float, bc2: float, grad_scale: float, extra_sumsq):
        """Returns (gradient norm, clip coefficient) — device views on CUDA. `extra_sumsq`
        is the squared norm of the replicated small-parameter gradients."""
        cfg = engine.cfg
        if self.mode != "fused":
            return self._collective_step(engine, lr, bc1, bc2, grad_scale, extra_sumsq)
        self._ensure_reduced(engine)
        overlapped = self._bucket_epoch is not None
        if overlapped:
            self._bucket_epoch = None          # the buckets of this step are in `_reduced` already (see reduce_bucket)
        else:
            self.epoch += 1
        native.call("sb_dp_update_step" if overlapped else "sb_dp_fused_step",
                    self.peer_ptrs("grads"), self.peer_ptrs("params"), self.peer_ptrs("sig"),
                    self._reduced.data_ptr(), engine.master.data_ptr(), engine.exp_avg.data_ptr(),
                    engine.exp_avg_sq.data_ptr(), self._scratch.data_ptr(), engine.rank * engine.shard,
                    engine.shard, self.rank, self.world_size, self.epoch, grad_scale, cfg.max_grad_norm, lr,
                    cfg.beta1, cfg.beta2, cfg.eps, cfg.weight_decay, bc1, bc2, extra_sumsq.data_ptr(),
                    engine.adamw_numel if engine.muon is not None else -1,
                    self._mc_ptrs.get("grads", 0) if self.multimem else None,
                    self._mc_ptrs.get("params", 0) if self.multimem else None, native.stream())
        return self._scratch[3], self._scratch[4:]

    def _ensure_reduced(self, engine) -> None:
        if self._reduced is None:
            self._reduced = torch.empty(engine.shard, device=self.device, dtype=torch.float32)

    # ------------------------------------------------------------------ reduce-scatter overlapped with backward
    def begin_bucketed_step(self, engine) -> bool:
        """Opens the step whose reduce-scatter runs bucket by bucket during its last backward pass. Returns
        False (and does nothing) outside the fused mode."""
        if self.mode != "fused":
            return False
        self._ensure_reduced(engine)
        self.epoch += 1
        self._bucket_epoch = self.epoch
        return True

    def reduce_bucket(self, engine, bucket: int, lo: int, hi: int, publish: bool, ctas: int, stream: int) -> None:
        """Launches the reduction of flat range [lo, hi) on `stream` (a raw handle). Every rank calls it for
        every bucket of the step in the same order; `publish` on the last one."""
        native.call("sb_dp_bucket_reduce", self.peer_ptrs("grads"), self.peer_ptrs("sig"), self._reduced.data_ptr(),
                    self._scratch.data_ptr(), engine.rank * engine.shard, engine.shard, lo, hi, bucket,
                    1 if publish else 0, self.rank, self.world_size, self._bucket_epoch,
                    self._mc_ptrs.get("grads", 0) if self.multimem else None, ctas, stream)

    def check_step(self) -> None:
        """Host side of the kernels' bounded waits; call after a step's norm has been read (the stream is
        idle then). A peer that was late or gone makes `sb_dp_fused_step` give up its waits, apply nothing
        and set bit 2 of the device error word: raise `RankFailure` here, before the step can be sealed
        into a checkpoint."""
        if self.mode != "fused":
            return
        word = native.read_error_flag()
        if word:
            from .health import RankFailure
            raise RankFailure([], f"device error word {word:#x} after data-parallel step {self.epoch} "
                                  "(bit 2: a peer's flag did not arrive in time; the update was skipped)")

    def all_gather(self, shard: torch.Tensor) -> torch.Tensor:
        """Concatenation of every rank's `shard` (same length everywhere), in rank order."""
        if dist.get_backend(self.group) == "gloo":
            parts = [torch.empty_like(shard) for _ in range(self.world_size)]
            dist.all_gather(parts, shard.contiguous(), group=self.group)
            return torch.cat(parts)
        full = torch.empty(shard.numel() * self.world_size, device=shard.device, dtype=shard.dtype)
        dist.all_gather_into_tensor(full, shard.contiguous(), group=self.group)
        return full

    def gather_reduced(self, engine) -> torch.Tensor:
        """The summed (unscaled) fp32 gradients of the whole flat buffer, rebuilt from the
        shards the last step reduced. Muon needs whole matrices, which the sharded step
        never materialises on one rank."""
        return self.all_gather(self._reduced if self.mode == "fused" else self._last_shard)

    def _collective_step(self, engine, lr, bc1, bc2, grad_scale, extra_sumsq):
        """Library-collective baseline with identical math."""
        cfg = engine.cfg
        g = engine.grads_flat
        shard = torch.empty(engine.shard, device=g.device, dtype=torch.float32)
        if dist.get_backend(self.group) == "gloo":
            # gloo has no reduce_scatter_tensor: all-reduce then slice
            full = g.clone()
            dist.all_reduce(full, group=self.group)
            shard.copy_(full[engine.rank * engine.shard:(engine.rank + 1) * engine.shard])
        else:
            dist.reduce_scatter_tensor(shard, g, group=self.group)
        self._last_shard = shard
        sq = shard.pow(2).sum()
        dist.all_reduce(sq, group=self.group)
        norm = (sq + extra_sumsq.reshape(-1)[0]).sqrt() * grad_scale
        coef = torch.full((), grad_scale, device=g.device)
        if cfg.max_grad_norm > 0:
            coef = coef * (cfg.max_grad_norm / (norm + 1e-6)).clamp(max=1.0)
        # with Muon, AdamW stops at the first Muon-owned element of the flat buffer
        n_ad = engine.shard
        if engine.muon is not None:
            n_ad = max(0, min(engine.shard, engine.adamw_numel - engine.rank * engine.shard))
        gg = shard[:n_ad] * coef
        m_, v_, w_ = engine.exp_avg[:n_ad], engine.exp_avg_sq[:n_ad], engine.master[:n_ad]
        m_.mul_(cfg.beta1).add_(gg, alpha=1 - cfg.beta1)
        v_.mul_(cfg.beta2).addcmul_(gg, gg, value=1 - cfg.beta2)
        upd = (m_ / bc1) / ((v_ / bc2).sqrt() + cfg.eps)
        w_.mul_(1 - lr * cfg.weight_decay).add_(upd, alpha=-lr)
        new_shard = engine.master.to(engine.params_flat.dtype)
        if dist.get_backend(self.group) == "gloo":
            parts = [torch.empty_like(new_shard) for _ in range(self.world_size)]
            dist.all_gather(parts, new_shard, group=self.group)
            engine.params_flat.copy_(torch.cat(parts))
        else:
            dist.all_gather_into_tensor(engine.params_flat, new_shard, group=self.group)
        if g.is_cuda:
            return norm, coef.reshape(1)
        return norm, float(coef)
