"""Peer-memory reduction for the tensor-parallel decoder: the all-reduce after a
row-split layer, the residual add and the RMSNorm that follow it, as one launch of
`b200q_tp_allreduce_add_rmsnorm` per call site.

The reference routes `std.nn.parallel::all_reduce` through a one-shot kernel over
symmetric memory when the message is small and through NCCL otherwise
(python/linnet/src/linnet/torch/collectives.py:145-167).  This is the same idea with the
two ops that always follow it in a decoder layer folded in, and with every wait bounded.

Memory comes from `torch.distributed._symmetric_memory` (one allocation per rank, mapped
into every peer by `rendezvous`); the kernel uses plain peer stores and local loads only.
"""

from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from . import _lib


class PeerReduce:
    """`sites` independent call sites of up to `max_rows` x `hidden` bf16 partial sums each.

    Per call site: `partial(site, rows)` is the tensor this rank's row-split linear writes
    its partial result into; `add_rmsnorm(site, x, weight, eps)` then reduces the ranks'
    partials, adds the sum to `x` in place and returns `rms_norm(x) * weight`.  Every rank
    must visit the sites in the same order, and at least two different sites must alternate
    (a site's buffer is safe to rewrite once any other site's reduction has been issued).

    `protocol`: how the ranks exchange their rows.  "words": every 8-byte word carries two
    values and the call's epoch, nothing else orders the ranks (`b200q_tp_allreduce_add_rmsnorm`).
    "flags": plain bf16 rows, then one flag per source rank and row
    (`b200q_tp_allreduce_add_rmsnorm_flags`).  Default: "words" on 2 ranks, "flags" on more
    (measured on the 8B-shape decoder at batch 1: 1.54 against 1.60 ms per step on 2 GPUs,
    1.46 against 1.32 ms on 8).
    """

    def __init__(self, sites: int, max_rows: int, hidden: int, device: torch.device,
                 group: "dist.ProcessGroup | None" = None, protocol: str | None = None) -> None:
        # plain peer stores and local loads only: the allocation needs no NVLink multicast binding
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm

        if sites < 2:
            raise ValueError("PeerReduce needs at least two call sites")
        group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if not 2 <= self.world <= 8:
            raise ValueError(f"PeerReduce runs on 2..8 ranks, not {self.world}")
        self.protocol = protocol or ("words" if self.world <= 2 else "flags")
        if self.protocol not in ("words", "flags"):
            raise ValueError(f"PeerReduce: unknown protocol {self.protocol!r}")
        self.sites, self.max_rows, self.hidden, self.device = sites, max_rows, hidden, device
        if self.protocol == "words":
            # per site: a receive area [source rank][max_rows][hidden / 2] words of (2 bf16, epoch)
            self.slot_elems = max_rows * hidden // 2
            self.area_bytes = self.world * self.slot_elems * 8
            self.flag_bytes = 0
        else:
            # per site: a receive area [source rank][max_rows][hidden] bf16; flags [source rank][max_rows] u32
            self.slot_elems = max_rows * hidden
            self.area_bytes = self.world * self.slot_elems * 2
            self.flag_bytes = self.world * max_rows * 4
        self.memory = symm.empty(sites * (self.area_bytes + self.flag_bytes), dtype=torch.uint8, device=device)
        self.memory.zero_()
        self.handle = symm.rendezvous(self.memory, group=group)
        self.bases = [int(p) for p in self.handle.buffer_ptrs]
        # "words": this rank's partial sums (local; rewritten before every reduction, in stream order)
        self.own = (torch.empty(max_rows, hidden, dtype=torch.bfloat16, device=device)
                    if self.protocol == "words" else None)
        # epoch and done counters per site, one error word
        self.state = torch.zeros(2 * sites + 1, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        dist.barrier(group=group)  # nobody stores into an area before every rank has zeroed its own
        int64s = ctypes.c_int64 * self.world
        self._areas = [int64s(*[b + s * self.area_bytes for b in self.bases]) for s in range(sites)]
        flags0 = sites * self.area_bytes
        self._flags = [int64s(*[b + flags0 + s * self.flag_bytes for b in self.bases]) for s in range(sites)]

    def partial(self, site: int, rows: int) -> torch.Tensor:
        """Where the row-split linear of a call site writes this rank's partial sums, `[rows,
        hidden]` bf16: "words" -- one local buffer for every site (read by the reduction that
        follows in the stream before the next linear writes it); "flags" -- this rank's own
        slot of the site's receive area (a view of the symmetric memory)."""
        if not 0 <= site < self.sites or not 0 < rows <= self.max_rows:
            raise ValueError(f"PeerReduce: site {site} / rows {rows} outside {self.sites} sites of {self.max_rows} rows")
        if self.protocol == "words":
            return self.own[:rows]
        start = site * self.area_bytes + self.rank * self.slot_elems * 2
        return self.memory[start:start + rows * self.hidden * 2].view(torch.bfloat16).view(rows, self.hidden)

    def add_rmsnorm(self, site: int, x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
        rows, hidden = x.shape
        if hidden != self.hidden or not 0 < rows <= self.max_rows or not 0 <= site < self.sites:
            raise ValueError("PeerReduce.add_rmsnorm: shape or site outside what was allocated")
        if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or not x.is_contiguous():
            raise ValueError("PeerReduce.add_rmsnorm: contiguous bf16 tensors only")
        y = torch.empty_like(x)
        state = self.state.data_ptr()
        counters = (state + 4 * site, state + 4 * (self.sites + site), state + 8 * self.sites)
        tail = (x.data_ptr(), weight.contiguous().data_ptr(), y.data_ptr(), rows, hidden, float(eps),
                torch.cuda.current_stream(self.device).cuda_stream)
        lib = _lib.load()
        if self.protocol == "words":
            _lib.check(lib.b200q_tp_allreduce_add_rmsnorm(
                ctypes.addressof(self._areas[site]), self.slot_elems, self.own.data_ptr(), self.world, self.rank,
                *counters, *tail))
        else:
            _lib.check(lib.b200q_tp_allreduce_add_rmsnorm_flags(
                ctypes.addressof(self._areas[site]), ctypes.addressof(self._flags[site]), self.slot_elems,
                self.max_rows, self.world, self.rank, *counters, *tail))
        return y

    def error(self) -> int:
        """0, or 100 + r when a wait for rank r ran out (synchronises the device)."""
        return int(self.state[2 * self.sites].item())


ONE_SHOT_BYTES = 128 * 1024  # the reference's limit (python/linnet/src/linnet/parallel.py:53)


class OneShot:
    """A group's buffers for the small-message all-reduce, with the reference's interface
    (`OneShot`, python/linnet/src/linnet/torch/collectives.py:56-103): built once per group by
    `collectives.prepare`, a collective call; `one_shot(x)` returns the sum of `x` over the
    group's ranks.  `install()` puts this class in the reference's place, so a `Shards` card's
    `std.nn.parallel::all_reduce` runs `b200q_tp_allreduce` for bf16 / f16 messages up to
    128 KiB whose length is a multiple of 8, in eager code, compiled code and CUDA graphs;
    anything else goes to NCCL the way the reference sends what its kernel does not cover
    (collectives.py:159-167).  Sums are taken in f32 in rank order: every rank gets the same
    bits.  Every wait on a peer is bounded (`b200q_set_wait_limit_ns`)."""

    def __init__(self, group: "dist.ProcessGroup") -> None:
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm

        self.group = group
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if not 2 <= self.world <= 8:
            raise RuntimeError(f"the peer-memory all-reduce runs on 2..8 ranks, not {self.world}")
        # two call sites that alternate; per site [source rank][slot] words of (2 values, epoch)
        self.slot_words = ONE_SHOT_BYTES // 2 // 2
        self.area_bytes = self.world * self.slot_words * 8
        self.memory = symm.empty(2 * self.area_bytes, dtype=torch.uint8, device=self.device)
        self.memory.zero_()
        handle = symm.rendezvous(self.memory, group=group.group_name)
        bases = [int(p) for p in handle.buffer_ptrs]
        int64s = ctypes.c_int64 * self.world
        self._areas = [int64s(*[b + s * self.area_bytes for b in bases]) for s in range(2)]
        self.state = torch.zeros(5, dtype=torch.int32, device=self.device)  # 2 epochs, 2 done counters, error
        self.site = 0
        torch.cuda.synchronize(self.device)
        dist.barrier(group)  # nobody stores into an area before every rank has zeroed its own

    def covers(self, x: torch.Tensor) -> bool:
        return (x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and x.numel() % 8 == 0
                and 0 < x.numel() * x.element_size() <= ONE_SHOT_BYTES)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        if not self.covers(x):
            return self._library(x)
        x = x.contiguous()
        out = torch.empty_like(x)
        site, self.site = self.site, 1 - self.site
        state = self.state.data_ptr()
        _lib.check(_lib.load().b200q_tp_allreduce(
            ctypes.addressof(self._areas[site]), self.slot_words, x.data_ptr(), self.world, self.rank,
            state + 4 * site, state + 4 * (2 + site), state + 16, out.data_ptr(), x.numel(),
            _lib.BF16 if x.dtype == torch.bfloat16 else _lib.F16,
            torch.cuda.current_stream(self.device).cuda_stream))
        return out

    def _library(self, x: torch.Tensor) -> torch.Tensor:
        """f32, odd lengths: the group's own backend, as the reference does past its kernel."""
        if torch.compiler.is_compiling() or torch.cuda.is_current_stream_capturing():
            from torch.distributed import _functional_collectives as funcol

            return funcol.all_reduce(x, "sum", self.group)
        out = x.clone(memory_format=torch.contiguous_format)
        dist.all_reduce(out, group=self.group)
        return out

    def error(self) -> int:
        """0, or 100 + r when a wait for rank r ran out (synchronises the device)."""
        return int(self.state[4].item())
