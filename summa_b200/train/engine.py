"""Training engine: flat parameter / gradient buffers, fused optimizer step,
data-parallel sharding.

Layout (per rank):
  * `params`  — one flat bf16 buffer holding every compute weight; the model's
    parameters are views into it.
  * `grads`   — one flat fp32 buffer; each parameter gets a `main_grad` view, and the
    weight-gradient GEMMs accumulate straight into it (TMA reduce-add), so gradient
    accumulation costs no extra pass.
  * `master`, `exp_avg`, `exp_avg_sq` — fp32, only for this rank's shard of the flat
    range (ZeRO-1 style).
With data parallelism both flat buffers live in symmetric memory: the fused kernel
in `summa_b200.parallel.dp` reads every peer's gradients for this rank's shard over
NVLink, reduces, clips, applies AdamW and writes the new bf16 weights into every
peer's parameter buffer — reduce-scatter, optimizer and all-gather in one launch.

Reference behaviour reproduced: AdamW(β 0.9/0.95, eps 1e-8, wd) with a global L2
gradient-norm clip before the update (`summa-train/src/trainer.rs:1123-1129,
1952-1975`, `summa-train/src/main.rs:667-694`).
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch
import torch.nn as nn

from ..ops import native


@dataclass
class OptimConfig:
    lr: float = 3e-4
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    weight_decay: float = 0.1
    max_grad_norm: float = 1.0       # <= 0 disables clipping


def _align(n: int, a: int) -> int:
    return (n + a - 1) // a * a


class FlatTrainEngine:
    """Owns the flat buffers of a model and performs optimizer steps.

    `dp` is an optional `summa_b200.parallel.dp.DataParallelGroup`; without it the
    engine runs single-device with the same buffers and the fused AdamW kernel.

    Parameters are split into two flat groups. Matrices (rank >= 2, the GEMM operands)
    live in the big `param_dtype` (bf16) buffer with fp32 master copies and are sharded
    under data parallelism. Everything numerically delicate and tiny — norm gains,
    biases, depthwise conv taps, `a_log`, `D` — stays fp32 in a second flat buffer that
    is replicated: its gradients are all-reduced and every rank applies the same update.
    Parameters marked `_sb_local` (expert shards under expert parallelism) form a third
    group that is never reduced: each rank owns them outright, with full optimizer state;
    only their squared gradient norm is summed over the ranks for the global clip.
    """

    def __init__(self, model: nn.Module, cfg: OptimConfig, dp=None, param_dtype=torch.bfloat16, muon: bool = False,
                 exclude=None):
        """`exclude(name) -> bool`: parameters that another optimizer owns (the memory tiers' banks);
        they stay out of the flat buffers, the norm and the step."""
        self.model = model
        self.cfg = cfg
        self.dp = dp
        self.step_count = 0
        self.muon = None
        self.extra_state = None          # optional callable -> {name: tensor} stored with the optimizer state
        self.loaded_extra = {}
        params = [(n, p) for n, p in model.named_parameters()
                  if p.requires_grad and not (exclude is not None and exclude(n))]
        self._managed = [p for _, p in params]
        self.device = params[0][1].device
        world = dp.world_size if dp is not None else 1
        rank = dp.rank if dp is not None else 0
        self.rank, self.world = rank, world

        def is_big(name, p):
            return p.dim() >= 2 and not name.endswith("a_log") and ".conv1d." not in name

        local = [(n, p) for n, p in params if getattr(p, "_sb_local", False)]
        params = [(n, p) for n, p in params if not getattr(p, "_sb_local", False)]
        big = [(n, p) for n, p in params if is_big(n, p)]
        small = [(n, p) for n, p in params if not is_big(n, p)]
        muon_names = set(model.muon_parameter_names()) if (muon and hasattr(model, "muon_parameter_names")) else set()
        # Muon-owned matrices go last so the flat AdamW pass (and its weight decay) can stop before them
        big = [x for x in big if x[0] not in muon_names] + [x for x in big if x[0] in muon_names]
        self.names = [n for n, _ in big]
        self.small_names = [n for n, _ in small]
        # each parameter starts on a 16-byte boundary of the bf16 buffer (TMA base alignment)
        offsets, total = [], 0
        for _, p in big:
            offsets.append(total)
            total += _align(p.numel(), 8)
        self.numel = total
        first_muon = next((o for (n, _), o in zip(big, offsets) if n in muon_names), total)
        self.adamw_numel = first_muon            # AdamW covers [0, adamw_numel)
        self.padded = _align(max(total, 1), world * 1024)
        self.shard = self.padded // world
        if dp is not None:
            self.params_flat = dp.alloc_symmetric(self.padded, param_dtype, "params")
            self.grads_flat = dp.alloc_symmetric(self.padded, torch.float32, "grads")
        else:
            self.params_flat = torch.zeros(self.padded, device=self.device, dtype=param_dtype)
            self.grads_flat = torch.zeros(self.padded, device=self.device, dtype=torch.float32)
        self.offsets: Dict[str, int] = {}
        with torch.no_grad():
            for (name, p), off in zip(big, offsets):
                n = p.numel()
                self.params_flat[off:off + n].copy_(p.detach().reshape(-1).to(param_dtype))
                p.data = self.params_flat[off:off + n].view(p.shape)
                p.main_grad = self.grads_flat[off:off + n].view(p.shape)
                self.offsets[name] = off
        lo = rank * self.shard
        self.master = self.params_flat[lo:lo + self.shard].float().clone()
        self.exp_avg = torch.zeros(self.shard, device=self.device, dtype=torch.float32)
        self.exp_avg_sq = torch.zeros(self.shard, device=self.device, dtype=torch.float32)
        # ---- small fp32 group (replicated)
        s_offsets, s_total = [], 0
        for _, p in small:
            s_offsets.append(s_total)
            s_total += _align(p.numel(), 4)
        self.small_numel = s_total
        n_small = max(s_total, 4)
        self.small_params = torch.zeros(n_small, device=self.device, dtype=torch.float32)
        self.small_grads = torch.zeros(n_small, device=self.device, dtype=torch.float32)
        self.small_exp_avg = torch.zeros(n_small, device=self.device, dtype=torch.float32)
        self.small_exp_avg_sq = torch.zeros(n_small, device=self.device, dtype=torch.float32)
        self.small_offsets: Dict[str, int] = {}
        with torch.no_grad():
            for (name, p), off in zip(small, s_offsets):
                n = p.numel()
                self.small_params[off:off + n].copy_(p.detach().reshape(-1).float())
                p.data = self.small_params[off:off + n].view(p.shape)
                p.main_grad = self.small_grads[off:off + n].view(p.shape)
                self.small_offsets[name] = off
        # ---- rank-local group (expert shards): bf16 params, fp32 grads, unsharded state
        self.local_names = [n for n, _ in local]
        l_offsets, l_total = [], 0
        for _, p in local:
            l_offsets.append(l_total)
            l_total += _align(p.numel(), 8)
        self.local_numel = l_total
        if l_total:
            self.local_params = torch.zeros(l_total, device=self.device, dtype=param_dtype)
            self.local_grads = torch.zeros(l_total, device=self.device, dtype=torch.float32)
            with torch.no_grad():
                for (name, p), off in zip(local, l_offsets):
                    n = p.numel()
                    self.local_params[off:off + n].copy_(p.detach().reshape(-1).to(param_dtype))
                    p.data = self.local_params[off:off + n].view(p.shape)
                    p.main_grad = self.local_grads[off:off + n].view(p.shape)
            self.local_master = self.local_params.float().clone()
            self.local_exp_avg = torch.zeros(l_total, device=self.device, dtype=torch.float32)
            self.local_exp_avg_sq = torch.zeros(l_total, device=self.device, dtype=torch.float32)
        self._scratch = torch.zeros(8, device=self.device, dtype=torch.float32)
        # Squared norm of gradients that live outside the flat buffers (memory-tier scopes), in the buffers' own units
        # (summed over ranks and micro-batches). Set before `step`, consumed by it: it joins the ONE global norm the
        # clip coefficient is derived from (`summa-train/src/main.rs:667-694`).
        self.extra_sumsq: Optional[torch.Tensor] = None
        if muon:
            from .muon import BatchedMuon
            self.muon = BatchedMuon(self, [n for n in self.names if n in muon_names])
        if dp is not None:
            # Opt-in. Shards are contiguous ranges of the flat buffer, so the rank that owns the range whose
            # gradients finish last (embeddings, first blocks) still has its whole reduction after the backward
            # pass and every rank waits for its norm: measured on 8 GPUs (llama-350m) the overlapped form is no
            # faster than the one-launch reduce-scatter (57.4 ms) and, with few CTAs per bucket, slower (62.1 ms).
            if os.environ.get("SUMMA_DP_OVERLAP", "0") == "1":
                self.enable_overlap()
            dp.barrier()

    # ------------------------------------------------------------------ reduce-scatter overlapped with backward
    def enable_overlap(self, n_buckets: int = 8, ctas: int = 8) -> bool:
        """Data parallelism, fused mode: cut the block matrices of the flat gradient buffer into `n_buckets`
        groups of consecutive blocks and reduce each group over the ranks on a side stream as soon as the last
        backward pass of a step has left it (`Transformer.grad_ready_hook`), with `ctas` CTAs next to the
        backward GEMMs. What no block owns (embeddings, output head) and whatever was not reached is reduced
        at the step. Returns False when the model or the group does not support it."""
        import re
        layers = getattr(self.model, "layers", None)
        if self.dp is None or getattr(self.dp, "mode", "") != "fused" or layers is None or not self.grads_flat.is_cuda:
            return False
        L = len(layers)
        params = dict(self.model.named_parameters())
        per_block = {i: [] for i in range(L)}
        for name in self.names:
            m = re.match(r"layers\.(\d+)\.", name)
            if m is not None:
                off = self.offsets[name]
                per_block[int(m.group(1))].append((off, off + _align(params[name].numel(), 8), params[name]))
        group = -(-L // max(1, n_buckets))
        jobs, taken = [], []                       # job: (blocks, lo, hi); one kernel launch each
        for b0 in range(0, L, group):
            blocks = frozenset(range(b0, min(L, b0 + group)))
            spans = sorted((lo, hi) for i in blocks for lo, hi, _ in per_block[i])
            merged = []
            for lo, hi in spans:
                if merged and merged[-1][1] == lo:
                    merged[-1][1] = hi
                else:
                    merged.append([lo, hi])
            jobs += [(blocks, lo, hi) for lo, hi in merged]
            taken += merged
        rest, at = [], 0
        for lo, hi in sorted(map(tuple, taken)):
            if lo > at:
                rest.append((at, lo))
            at = max(at, hi)
        if at < self.padded:
            rest.append((at, self.padded))
        if not jobs or len(jobs) + len(rest) > 60:
            return False
        self._ov_jobs = [dict(id=k, blocks=b, lo=lo, hi=hi, launched=False) for k, (b, lo, hi) in enumerate(jobs)]
        self._ov_rest = [dict(id=len(jobs) + k, lo=lo, hi=hi) for k, (lo, hi) in enumerate(rest)]
        self._ov_block_params = {i: [p for _, _, p in per_block[i]] for i in range(L)}
        self._ov_bucketed = {id(p) for i in range(L) for p in self._ov_block_params[i]}
        self._ov_ctas = ctas
        self._ov_side = torch.cuda.Stream(device=self.device)
        self._ov_hook = _OverlapHook(self)
        self.model.grad_ready_hook = self._ov_hook
        return True

    def arm_overlap(self) -> None:
        """Call before the forward pass of a step's LAST micro-batch: its backward pass hands finished buckets
        to the reduce-scatter. A no-op without `enable_overlap`."""
        hook = getattr(self, "_ov_hook", None)
        if hook is None or hook.armed or not self.dp.begin_bucketed_step(self):
            return
        for j in self._ov_jobs:
            j["launched"] = False
        hook.arm(len(self.model.layers))

    def _ov_launch_ready(self, done) -> None:
        for j in self._ov_jobs:
            if j["launched"] or not j["blocks"] <= done:
                continue
            for i in j["blocks"]:                    # gradients that came through autograd's `.grad`
                for p in self._ov_block_params[i]:
                    if p.grad is not None:
                        p.main_grad.add_(p.grad.to(torch.float32).view_as(p.main_grad))
                        p.grad = None
            ev = torch.cuda.Event()
            ev.record()                              # the backward pass's stream, in the autograd thread
            self._ov_side.wait_event(ev)
            self.dp.reduce_bucket(self, j["id"], j["lo"], j["hi"], False, self._ov_ctas, self._ov_side.cuda_stream)
            j["launched"] = True

    def _ov_finish(self) -> None:
        """At the step: everything that was not reduced during the backward pass, on the step's stream."""
        hook = self._ov_hook
        hook.armed = False
        cur = torch.cuda.current_stream()
        cur.wait_stream(self._ov_side)
        todo = [j for j in self._ov_jobs if not j["launched"]] + self._ov_rest
        if not todo:
            todo = [dict(id=63, lo=0, hi=0)]         # nothing left to reduce: the launch only publishes the norm
        for k, j in enumerate(todo):
            self.dp.reduce_bucket(self, j["id"], j["lo"], j["hi"], k == len(todo) - 1, 0, cur.cuda_stream)

    # ------------------------------------------------------------------ gradient plumbing
    def zero_grad(self) -> None:
        self.grads_flat.zero_()
        self.small_grads.zero_()
        if self.local_numel:
            self.local_grads.zero_()
        for p in self._managed:
            p.grad = None

    @torch.no_grad()
    def layer_gradient_norms(self, num_layers: int, grad_scale: float = 1.0) -> List[float]:
        """Pre-clip L2 norm of this rank's accumulated gradient per transformer layer (parameters named
        `layers.<i>.`), for the opt-in `layer_gradient_norms` field of the optimization record
        (`summa-train/src/trainer.rs:1941-1950`). One device reduction per layer group, one host read. Under data
        parallelism the gradients are those of this rank before the reduction; the caller combines ranks."""
        import re
        sq = torch.zeros(max(num_layers, 1), device=self.device, dtype=torch.float32)
        self.fold_autograd_grads()
        for name, p in self.model.named_parameters():
            m = re.match(r"(?:module\.)?layers\.(\d+)\.", name)
            g = getattr(p, "main_grad", None)
            if m is None or g is None or int(m.group(1)) >= num_layers:
                continue
            sq[int(m.group(1))] += g.float().pow(2).sum()
        return [float(v) for v in (sq.sqrt() * grad_scale).tolist()[:num_layers]]

    def fold_autograd_grads(self) -> None:
        """Gradients that arrived through autograd's `.grad` (ops without a fused
        main-grad epilogue) are added into the flat fp32 buffers."""
        armed = getattr(self, "_ov_hook", None) is not None and self._ov_hook.armed
        for p in self._managed:
            if p.grad is not None and hasattr(p, "main_grad"):
                if armed and id(p) in self._ov_bucketed:
                    raise RuntimeError("a block parameter's gradient arrived after its bucket had been reduced "
                                       "(overlapped reduce-scatter needs one forward pass per block and micro-batch)")
                p.main_grad.add_(p.grad.to(torch.float32).view_as(p.main_grad))
                p.grad = None

    # ------------------------------------------------------------------ quantisation-aware training
    @torch.no_grad()
    def begin_quantized_window(self, fmt: str, names) -> int:
        """The compute copies of `names` take dequant(quant(w)) until the optimizer step that ends
        this accumulation window. Gradients reach the fp32 masters unchanged, which is the
        straight-through estimator `w + (q(w) - w).detach()` (`summa-train/src/quantization.rs:792-932`):
        the step rewrites every compute copy from its master. Parameters that are their own fp32
        master (the small group) are saved here and put back by `end_quantized_window`."""
        from .quantization import fake_quant_values
        params = dict(self.model.named_parameters())
        self._qat_saved = {}
        for n in names:
            p = params[n]
            if n in self.small_offsets:
                self._qat_saved[n] = p.detach().clone()
            p.data.copy_(fake_quant_values(p.data, fmt))
        return len(names)

    @torch.no_grad()
    def end_quantized_window(self) -> None:
        """Call before `step`: the self-mastered parameters get their full-precision values back."""
        params = dict(self.model.named_parameters())
        for n, saved in getattr(self, "_qat_saved", {}).items():
            params[n].data.copy_(saved)
        self._qat_saved = {}

    # ------------------------------------------------------------------ step
    def step(self, lr: Optional[float] = None, grad_scale: float = 1.0) -> torch.Tensor:
        """Clip + AdamW over the flat buffers. Returns the (pre-clip) global gradient
        norm as a device scalar. `grad_scale` multiplies gradients first (e.g. 1/ga)."""
        self.fold_autograd_grads()
        cfg = self.cfg
        lr = cfg.lr if lr is None else lr
        self.step_count += 1
        bc1 = 1.0 - cfg.beta1 ** self.step_count
        bc2 = 1.0 - cfg.beta2 ** self.step_count
        g, sg, sc = self.grads_flat, self.small_grads, self._scratch
        cuda = g.is_cuda
        if self.dp is not None:
            # the summed rank gradients become the gradient of the global-batch mean
            grad_scale = grad_scale / self.world
            self.dp.all_reduce(sg)
        if cuda:
            sc.zero_()
            native.call("sb_sumsq", sg.data_ptr(), sg.numel(), sc[5:].data_ptr(), native.stream())
            if self.local_numel:
                # rank-local gradients: only their squared norm crosses ranks
                native.call("sb_sumsq", self.local_grads.data_ptr(), self.local_numel, sc[6:].data_ptr(), native.stream())
                if self.dp is not None:
                    self.dp.all_reduce(sc[6:7])
                sc[5] += sc[6]
            if self.extra_sumsq is not None:
                sc[5] += self.extra_sumsq.to(device=sc.device, dtype=torch.float32)
                self.extra_sumsq = None
            if self.dp is not None:
                if getattr(self, "_ov_hook", None) is not None and self._ov_hook.armed:
                    self._ov_finish()
                norm, coef_ptr = self.dp.fused_step(self, lr, bc1, bc2, grad_scale, sc[5:])
                if self.muon is not None:
                    self.muon.step(lr * 20.0, coef_ptr, self.dp.gather_reduced(self))
            else:
                native.call("sb_sumsq", g.data_ptr(), self.numel, sc.data_ptr(), native.stream())
                norm = (sc[0] + sc[5]).sqrt() * grad_scale
                # clip coefficient stays on the device: no host sync in the step
                if cfg.max_grad_norm > 0:
                    coef = (cfg.max_grad_norm / (norm + 1e-6)).clamp(max=1.0) * grad_scale
                else:
                    coef = torch.full((), grad_scale, device=g.device)
                sc[1] = coef
                coef_ptr = sc[1:]
                if self.muon is not None:
                    self.muon.step(lr * 20.0, coef_ptr)     # zeroes the gradients it consumed
                native.call("sb_adamw", self.master.data_ptr(), self.exp_avg.data_ptr(), self.exp_avg_sq.data_ptr(),
                            g.data_ptr(), self.params_flat.data_ptr(),
                            self.padded if self.muon is None else max(self.adamw_numel, 1), coef_ptr.data_ptr(), lr,
                            cfg.beta1, cfg.beta2, cfg.eps, cfg.weight_decay, bc1, bc2, native.stream())
            native.call("sb_adamw", self.small_params.data_ptr(), self.small_exp_avg.data_ptr(),
                        self.small_exp_avg_sq.data_ptr(), sg.data_ptr(), None, sg.numel(), coef_ptr.data_ptr(), lr,
                        cfg.beta1, cfg.beta2, cfg.eps, cfg.weight_decay, bc1, bc2, native.stream())
            if self.local_numel:
                native.call("sb_adamw", self.local_master.data_ptr(), self.local_exp_avg.data_ptr(),
                            self.local_exp_avg_sq.data_ptr(), self.local_grads.data_ptr(), self.local_params.data_ptr(),
                            self.local_numel, coef_ptr.data_ptr(), lr, cfg.beta1, cfg.beta2, cfg.eps, cfg.weight_decay,
                            bc1, bc2, native.stream())
            return norm
        # CPU path (same math in PyTorch)
        small_sq = sg.pow(2).sum()
        if self.local_numel:
            lsq = self.local_grads.pow(2).sum().reshape(1)
            if self.dp is not None:
                self.dp.all_reduce(lsq)
            small_sq = small_sq + lsq[0]
        if self.extra_sumsq is not None:
            small_sq = small_sq + self.extra_sumsq.to(device=sg.device, dtype=small_sq.dtype)
            self.extra_sumsq = None
        if self.dp is not None:
            norm, coef = self.dp.fused_step(self, lr, bc1, bc2, grad_scale, small_sq)
            if self.muon is not None:
                self.muon.step(lr * 20.0, coef, self.dp.gather_reduced(self))
        else:
            norm = (g[:self.numel].pow(2).sum() + small_sq).sqrt() * grad_scale
            coef = grad_scale
            if cfg.max_grad_norm > 0:
                coef = float(min(1.0, cfg.max_grad_norm / (norm.item() + 1e-6))) * grad_scale
            if self.muon is not None:
                self.muon.step(lr * 20.0, coef)
            n_ad = self.padded if self.muon is None else self.adamw_numel
            _adamw_torch(self.master[:n_ad], self.exp_avg[:n_ad], self.exp_avg_sq[:n_ad], g[:n_ad] * coef, lr, cfg,
                         bc1, bc2)
            self.params_flat[:n_ad].copy_(self.master[:n_ad].to(self.params_flat.dtype))
        _adamw_torch(self.small_params, self.small_exp_avg, self.small_exp_avg_sq, sg * coef, lr, cfg, bc1, bc2)
        if self.local_numel:
            _adamw_torch(self.local_master, self.local_exp_avg, self.local_exp_avg_sq, self.local_grads * coef, lr, cfg,
                         bc1, bc2)
            self.local_params.copy_(self.local_master.to(self.local_params.dtype))
        return norm

    # ------------------------------------------------------------------ state
    def state_dict(self) -> dict:
        return {"step": self.step_count, "master": self.master, "exp_avg": self.exp_avg,
                "exp_avg_sq": self.exp_avg_sq, "small_exp_avg": self.small_exp_avg,
                "small_exp_avg_sq": self.small_exp_avg_sq, "rank": self.rank, "world": self.world,
                "numel": self.numel, "offsets": dict(self.offsets), "small_offsets": dict(self.small_offsets)}

    def load_state_dict(self, sd: dict) -> None:
        self.step_count = int(sd["step"])
        self.master.copy_(sd["master"])
        self.exp_avg.copy_(sd["exp_avg"])
        self.exp_avg_sq.copy_(sd["exp_avg_sq"])
        self.small_exp_avg.copy_(sd["small_exp_avg"])
        self.small_exp_avg_sq.copy_(sd["small_exp_avg_sq"])
        lo = self.rank * self.shard
        self.params_flat[lo:lo + self.shard].copy_(self.master.to(self.params_flat.dtype))

    def _full(self, shard: torch.Tensor) -> torch.Tensor:
        """The whole flat tensor (unpadded) from this rank's shard; a collective under data parallelism."""
        return (shard if self.dp is None else self.dp.all_gather(shard))[:self.numel]

    def _take_shard(self, dst: torch.Tensor, full: torch.Tensor) -> None:
        lo = self.rank * self.shard
        hi = min(lo + self.shard, full.numel())
        dst.zero_()
        if hi > lo:
            dst[:hi - lo].copy_(full[lo:hi].to(dst.device))

    def pack_state(self):
        """(adamw container bytes, muon container bytes) for a checkpoint generation. The flat
        tensors are stored whole and unpadded, so a checkpoint resumes on any number of ranks;
        under data parallelism every rank must call this (the shards are gathered) and all ranks
        return the same bytes."""
        from .checkpoint import pack_tensors
        master = self._full(self.master)
        if self.muon is not None and self.muon.own_master:
            master = master.clone()
            for n, m in self.muon.master.items():       # the sharded master never sees Muon's updates
                master[self.offsets[n]:self.offsets[n] + m.numel()] = m.reshape(-1)
        tensors = {"master": master, "exp_avg": self._full(self.exp_avg), "exp_avg_sq": self._full(self.exp_avg_sq),
                   "small_exp_avg": self.small_exp_avg, "small_exp_avg_sq": self.small_exp_avg_sq}
        if self.local_numel:             # rank-local (expert) group: each rank's container carries its own
            tensors.update({"local_master": self.local_master, "local_exp_avg": self.local_exp_avg,
                            "local_exp_avg_sq": self.local_exp_avg_sq})
        if self.extra_state is not None:
            tensors.update({"extra." + k: v for k, v in self.extra_state().items()})
        adamw = pack_tensors(tensors, {"step": float(self.step_count), "rank": float(self.rank), "world": float(self.world)},
                             {"layout": "flat-v2"})
        muon = pack_tensors(self.muon.state_tensors() if self.muon is not None else {}, {}, {})
        return adamw, muon

    def load_packed(self, adamw: bytes, muon: bytes) -> None:
        from .checkpoint import unpack_tensors
        t, sc, _ = unpack_tensors(adamw)
        self.loaded_extra = {k[len("extra."):]: v for k, v in t.items() if k.startswith("extra.")}
        if t:
            self.step_count = int(sc.get("step", 0))
            for name in ("master", "exp_avg", "exp_avg_sq"):
                self._take_shard(getattr(self, name), t[name])
            for name in ("small_exp_avg", "small_exp_avg_sq"):
                getattr(self, name).copy_(t[name].to(self.device))
            if self.muon is not None and self.muon.own_master:
                for n, m in self.muon.master.items():
                    off = self.offsets[n]
                    m.copy_(t["master"][off:off + m.numel()].view_as(m).to(m.device))
            if self.local_numel and "local_master" in t:
                for name in ("local_master", "local_exp_avg", "local_exp_avg_sq"):
                    getattr(self, name).copy_(t[name].to(self.device))
                self.local_params.copy_(self.local_master.to(self.local_params.dtype))
        if self.muon is not None:
            mt, _, _ = unpack_tensors(muon)
            self.muon.load_state_tensors(mt)

    def resync_from_model(self) -> None:
        """After weights were loaded into the model's (flat-buffer) parameters: restore the
        exact fp32 master from the optimizer state when present, else derive it."""
        lo = self.rank * self.shard
        if float(self.master.abs().sum()) == 0.0:
            self.master.copy_(self.params_flat[lo:lo + self.shard].float())
        else:
            self.params_flat[lo:lo + self.shard].copy_(self.master.to(self.params_flat.dtype))

    def resync_master(self) -> None:
        """Re-derive the fp32 master shard from the parameter buffer (after loading weights)."""
        lo = self.rank * self.shard
        self.master.copy_(self.params_flat[lo:lo + self.shard].float())


class _OverlapHook:
    """What `Transformer.forward_hidden` calls around each block while a step's last micro-batch is in flight:
    a block is done when every forward application of it has seen its backward."""

    def __init__(self, engine: "FlatTrainEngine"):
        self.engine = engine
        self.armed = False
        self.pending: Dict[int, int] = {}
        self.done = set()

    def arm(self, n_blocks: int) -> None:
        self.pending = {}
        self.done = set()
        self.armed = True

    def on_forward(self, i: int) -> None:
        self.pending[i] = self.pending.get(i, 0) + 1
        self.done.discard(i)

    def on_backward(self, i: int) -> None:
        if not self.armed:
            return
        self.pending[i] = self.pending.get(i, 1) - 1
        if self.pending[i] <= 0:
            self.done.add(i)
            self.engine._ov_launch_ready(self.done)


def _adamw_torch(p, m, v, g, lr, cfg, bc1, bc2):
    m.mul_(cfg.beta1).add_(g, alpha=1 - cfg.beta1)
    v.mul_(cfg.beta2).addcmul_(g, g, value=1 - cfg.beta2)
    upd = (m / bc1) / ((v / bc2).sqrt() + cfg.eps)
    p.mul_(1 - lr * cfg.weight_decay).add_(upd, alpha=-lr)


def train_step(model, engine: FlatTrainEngine, tokens: torch.Tensor, targets: torch.Tensor,
               lr: Optional[float] = None, grad_accum: int = 1):
    """One optimizer step over `grad_accum` micro-batches stacked on dim 0 of tokens.
    Returns (mean loss, gradient norm) as device scalars."""
    engine.zero_grad()
    micro = tokens.shape[0] // grad_accum
    total = None
    for i in range(grad_accum):
        t = tokens[i * micro:(i + 1) * micro]
        y = targets[i * micro:(i + 1) * micro]
        if i == grad_accum - 1:
            engine.arm_overlap()
        out = model.forward_loss(t, y, with_router=True)
        loss, aux = out
        (loss + aux).backward()
        total = loss.detach() if total is None else total + loss.detach()
    norm = engine.step(lr, grad_scale=1.0 / grad_accum)
    return total / grad_accum, norm


def checked_norm(engine: FlatTrainEngine, norm) -> float:
    """The step's gradient norm on the host (a synchronisation), followed by the failure checks
    that must happen before the step counts: a non-zero device error word under data parallelism
    (a bounded peer wait ran out and the fused step applied nothing) raises `RankFailure`."""
    value = float(norm)
    if engine.dp is not None and hasattr(engine.dp, "check_step"):
        engine.dp.check_step()
    return value
