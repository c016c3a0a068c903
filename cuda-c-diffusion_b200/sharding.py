"""Multi-GPU partitioning of the path: one process per GPU, `torch.distributed` for the plumbing.

What shards and how (no kernel reads another GPU's memory):

* norms, activations, skip merges, embeddings: independent per sample.  NHWC is
  sample-major, so a batch shard is a contiguous pointer range (`batch_shard`);
  no communication.
* dgamma / dbeta of GroupNorm / LayerNorm over a sharded batch: each rank holds
  partial sums of 2*C floats; one all-reduce (`allreduce_param_grads`).  In
  data-parallel training this rides with the gradient all-reduce.
* Adam + EMA: sharded by parameter range (`param_range`, 16-byte aligned cuts).
  m, v and the EMA shadow exist only for the local range; after the fused update
  the new parameters are all-gathered in place (`ShardedAdamEMA`).
* data-parallel training step: gradients are summed across ranks
  (`allreduce_gradients`) and the 1/world factor is folded into the update's
  `grad_scale`, so no separate scaling pass runs.

The update kernel is injected (`update_fn`) so that the partitioning logic can
be exercised with the gloo backend on CPU; the default is the CUDA entry point,
which raises without a GPU build.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch
import torch.distributed as dist


def batch_shard(n_samples: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous sample range [start, start+count) of `rank`; the first n % world ranks get one extra."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(n_samples, world)
    start = rank * base + min(rank, extra)
    return start, base + (1 if rank < extra else 0)


def param_range(n: int, rank: int, world: int, align: int = 4) -> tuple[int, int]:
    """Contiguous element range of a flat parameter vector owned by `rank`.  Cuts fall on
    multiples of `align` floats (16 bytes) so that every shard keeps 128-bit accesses; the
    ranges tile [0, n) exactly and the last ranks may be empty for tiny n."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    blocks = (n + align - 1) // align
    base, extra = divmod(blocks, world)
    b0 = rank * base + min(rank, extra)
    b1 = b0 + base + (1 if rank < extra else 0)
    return min(b0 * align, n), min(b1 * align, n)


def equal_param_range(n: int, world: int, align: int = 4) -> int:
    """Per-rank shard length when every rank must own the same number of elements (what an
    in-place all-gather needs): n is padded up to world * shard."""
    blocks = (n + align - 1) // align
    return ((blocks + world - 1) // world) * align


def allreduce_param_grads(*tensors: torch.Tensor, group=None) -> None:
    """Sum per-rank partial parameter gradients (dgamma, dbeta) in place."""
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        for t in tensors:
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)


def allreduce_gradients(flat_grad: torch.Tensor, group=None) -> float:
    """Data-parallel gradient exchange: sums `flat_grad` across ranks in place and returns the
    factor (1/world) the optimizer must apply as `grad_scale`."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world > 1:
        dist.all_reduce(flat_grad, op=dist.ReduceOp.SUM, group=group)
    return 1.0 / world


def _cuda_update(p, m, v, shadow, g, hyper):
    from . import ops
    ops.adam_ema_step_(p, m, v, shadow, g, hyper.lr, hyper.beta1, hyper.beta2, hyper.eps, hyper.bc1, hyper.bc2,
                       hyper.decay, hyper.grad_scale)


@dataclass
class AdamHyper:
    lr: float
    beta1: float
    beta2: float
    eps: float
    bc1: float
    bc2: float
    decay: float
    grad_scale: float = 1.0


class ShardedAdamEMA:
    """Fused Adam + EMA over a flat fp32 parameter vector sharded by parameter range.

    Every rank keeps the full (padded) parameter vector, but moments and the EMA shadow only
    for the contiguous range it owns.  `step` updates that range with one fused pass and
    all-gathers the new parameters in place (send buffer = own slice of the receive buffer).
    Bias corrections follow the reference host code (optimizer.c:62-64: bc = 1 - beta^t in fp32).

    This is the torch.distributed form used by the CPU (gloo) tests of the partitioning; the
    product form for one process per GPU is csrc/host/b200_sharded_optimizer.c (C, NCCL, with
    the exchange optionally fused into the update kernel as peer stores).
    """

    def __init__(self, params: torch.Tensor, lr, beta1=0.9, beta2=0.999, eps=1e-8, decay=0.999, group=None,
                 update_fn=None):
        assert params.dim() == 1 and params.dtype == torch.float32
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.n = params.numel()
        self.shard = equal_param_range(self.n, self.world)  # 16-byte aligned, the same on every rank
        padded = self.shard * self.world
        self.params = params if padded == self.n else torch.cat(
            [params, torch.zeros(padded - self.n, dtype=params.dtype, device=params.device)])
        self.lo, self.hi = self.rank * self.shard, (self.rank + 1) * self.shard
        self.m = torch.zeros(self.shard, dtype=torch.float32, device=params.device)
        self.v = torch.zeros_like(self.m)
        self.shadow = self.params[self.lo:self.hi].clone()
        self.lr, self.beta1, self.beta2, self.eps, self.decay = lr, beta1, beta2, eps, decay
        self.t = 0
        self.update_fn = update_fn or _cuda_update

    def local_params(self) -> torch.Tensor:
        return self.params[self.lo:self.hi]

    def hyper(self, grad_scale=1.0) -> AdamHyper:
        tt = np.float32(self.t)
        bc1 = float(np.float32(1.0) - np.power(np.float32(self.beta1), tt))
        bc2 = float(np.float32(1.0) - np.power(np.float32(self.beta2), tt))
        return AdamHyper(self.lr, self.beta1, self.beta2, self.eps, bc1, bc2, self.decay, grad_scale)

    def _grad_piece(self, grads, lo, hi):
        g = grads[lo:min(hi, grads.numel())] if lo < grads.numel() else grads[:0]
        if g.numel() < hi - lo:  # the padding tail has zero gradient
            g = torch.cat([g, torch.zeros(hi - lo - g.numel(), dtype=grads.dtype, device=grads.device)])
        return g.contiguous()

    def step(self, grads: torch.Tensor, grad_scale: float = 1.0, gather: bool = True) -> None:
        """`grads`: full (padded or unpadded) flat gradient; only the owned range is read."""
        self.t += 1
        self.update_fn(self.local_params(), self.m, self.v, self.shadow, self._grad_piece(grads, self.lo, self.hi),
                       self.hyper(grad_scale))
        if gather:
            self.all_gather()

    def all_gather(self) -> None:
        if self.world > 1:
            dist.all_gather_into_tensor(self.params, self.local_params(), group=self.group)

    def full_params(self) -> torch.Tensor:
        return self.params[:self.n]

    def gather_state(self):
        """Moments and shadow gathered to the unsharded layout (what a checkpoint stores per tensor)."""
        outs = []
        for t in (self.m, self.v, self.shadow):
            full = torch.empty(self.shard * self.world, dtype=t.dtype, device=t.device)
            if self.world > 1:
                dist.all_gather_into_tensor(full, t.contiguous(), group=self.group)
            else:
                full.copy_(t)
            outs.append(full[:self.n])
        return tuple(outs)
