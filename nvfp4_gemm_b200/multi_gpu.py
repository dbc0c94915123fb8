"""Column-parallel NVFP4 GEMM over the GPUs of one node (one process per GPU).

Only the large GEMM is partitioned.  Rank r holds all of ``a`` (+ its scales) and rows
[r*N/g, (r+1)*N/g) of ``b`` with the matching row blocks of the permuted ``sfb``; it computes
C[:, r*N/g:(r+1)*N/g] with the single-GPU kernel, and the fp16 column blocks are all-gathered with
NCCL over NVLink.  The output columns are independent, so the all-gather is the only exchange.

The all-gather wants contiguous per-rank chunks, but a column block is strided inside row-major C.
Each rank therefore computes into a contiguous staging block [rows, N/g], the gather lands as
[g][rows][N/g], and one HBM-bound kernel (``nvfp4_interleave_column_blocks``) writes [rows][N].
The rows are processed in panels so that the GEMM of panel i+1 overlaps the gather and the
re-layout of panel i (NCCL runs on the process group's own stream).

The reference has no multi-GPU code; this follows the operator contract of template.py:4-25 on
each rank.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class ColumnShard:
    rank: int
    world: int
    n_total: int

    @property
    def n_local(self) -> int:
        return self.n_total // self.world

    @property
    def begin(self) -> int:
        return self.rank * self.n_local

    @property
    def end(self) -> int:
        return self.begin + self.n_local


def plan_shard(n: int, world: int, rank: int) -> ColumnShard:
    """Equal column blocks; each must be whole 128-row scale blocks (the permuted SFB is sliced by block)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    if n % (128 * world):
        raise ValueError(f"N = {n} must be a multiple of 128 * world_size = {128 * world}")
    return ColumnShard(rank, world, n)


def shard_inputs(data, shard: ColumnShard):
    """Slice the full 7-tuple down to this rank's operands (views, nothing is copied):
    all of a/sfa, rows [begin, end) of b/sfb, row blocks [begin/128, end/128) of sfb_permuted."""
    a, b, sfa, sfb, sfa_perm, sfb_perm, c = data
    rb0, rb1 = shard.begin // 128, shard.end // 128
    return (a, b[shard.begin:shard.end], sfa, sfb[shard.begin:shard.end], sfa_perm, sfb_perm[:, :, rb0:rb1], c)


def row_panels(m: int, panels: int):
    """Split M into at most `panels` ranges of whole 256-row tiles."""
    tiles = (m + 255) // 256
    panels = max(1, min(panels, tiles))
    out, start = [], 0
    for p in range(panels):
        t = tiles // panels + (1 if p < tiles % panels else 0)
        end = min(m, start + t * 256)
        if end > start:
            out.append((start, end))
        start = end
    return out


def to_device_same_layout(t: torch.Tensor, device) -> torch.Tensor:
    """Copy a dense (possibly permuted) tensor to `device` byte for byte, keeping its strides: the
    permuted scale tensors are defined by their memory layout, which a logical copy could change."""
    raw = t.view(torch.uint8) if t.element_size() == 1 else t
    flat = torch.as_strided(raw, (t.numel(),), (1,), raw.storage_offset())
    moved = flat.to(device)
    out = torch.as_strided(moved, tuple(t.shape), tuple(t.stride()), 0)
    return out.view(t.dtype) if t.element_size() == 1 else out


def _default_gemm(panel_data):
    from .submission import custom_kernel
    return custom_kernel(panel_data)


def _default_interleave(src: torch.Tensor, dst: torch.Tensor, rows: int, n_local: int, blocks: int, dst_row_stride: int):
    from . import _lib
    lib = _lib.load()
    _lib.check(lib.nvfp4_interleave_column_blocks(src.data_ptr(), dst.data_ptr(), rows, n_local, blocks, dst_row_stride,
                                                  torch.cuda.current_stream(dst.device).cuda_stream))


class ColumnParallelGemm:
    """Reusable plan + buffers for one problem shape on one rank.

    ``gemm_fn`` and ``interleave_fn`` exist so that the host logic can be exercised on CPU ranks
    (gloo) with stand-ins; the defaults are the CUDA library.
    """

    def __init__(self, m: int, n: int, k: int, group=None, device=None, panels: int = 4,
                 gemm_fn: Optional[Callable] = None, interleave_fn: Optional[Callable] = None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.shard = plan_shard(n, self.world, self.rank)
        self.m, self.n, self.k = m, n, k
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.panels = row_panels(m, panels)
        self.gemm_fn = gemm_fn or _default_gemm
        self.interleave_fn = interleave_fn or _default_interleave
        nl = self.shard.n_local
        # staging [1][m][n_local] (the operator's c layout with l = 1) and gather target per panel
        self.staging = torch.empty((1, m, nl), dtype=torch.float16, device=self.device)
        self.gathered = [torch.empty((self.world, p1 - p0, nl), dtype=torch.float16, device=self.device)
                         for (p0, p1) in self.panels]

    def __call__(self, local_data, c_full: torch.Tensor) -> torch.Tensor:
        """local_data: this rank's 7-tuple (its ``c`` entry is ignored); c_full: [M, N, 1] fp16, row-major."""
        a, b, sfa, sfb, sfa_perm, sfb_perm, _ = local_data
        if a.shape[2] != 1:
            raise ValueError("the column-parallel path handles l = 1")
        nl = self.shard.n_local
        works = []
        for idx, (p0, p1) in enumerate(self.panels):
            rb0, rb1 = p0 // 128, (p1 + 127) // 128
            c_panel = self.staging[:, p0:p1, :].permute(1, 2, 0)          # [rows, n_local, 1]
            panel = (a[p0:p1], b, sfa[p0:p1], sfb, sfa_perm[:, :, rb0:rb1], sfb_perm, c_panel)
            self.gemm_fn(panel)
            works.append(dist.all_gather_into_tensor(self.gathered[idx].view(-1, nl), self.staging[0, p0:p1, :], group=self.group,
                                                     async_op=True))
            if idx > 0:
                self._finish_panel(idx - 1, works[idx - 1], c_full)
        self._finish_panel(len(self.panels) - 1, works[-1], c_full)
        return c_full

    def _finish_panel(self, idx: int, work, c_full: torch.Tensor):
        p0, p1 = self.panels[idx]
        work.wait()   # makes the current stream wait for the collective; the host does not block on CUDA
        dst = c_full[p0:p1]
        self.interleave_fn(self.gathered[idx], dst, p1 - p0, self.shard.n_local, self.world, c_full.stride(0))


def symmetric_output(m: int, n: int, device, group):
    """The full fp16 output [m * n] in symmetric memory, mapped into every rank's address space
    for PLAIN peer loads and stores: the buffer must not be bound to an NVLink multicast object
    (none of the kernels here use one, and a rank that dies while bound to one disturbs its
    peers).  Returns (tensor, rendezvous handle); raises if the binding could not be avoided."""
    import os
    os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "1"     # read by torch when the buffer is exchanged
    import torch.distributed._symmetric_memory as symm_mem
    c_sym = symm_mem.empty((m * n,), dtype=torch.float16, device=device)
    handle = symm_mem.rendezvous(c_sym, group)
    check_no_multicast(handle)
    return c_sym, handle


def check_no_multicast(handle) -> None:
    if int(getattr(handle, "multicast_ptr", 0) or 0) != 0:
        raise RuntimeError("the symmetric output buffer is bound to an NVLink multicast object although "
                           "TORCH_SYMM_MEM_DISABLE_MULTICAST=1 was set: set it in the environment before torch initialises "
                           "symmetric memory")


class FusedAllGatherGemm:
    """Column-parallel GEMM whose epilogue is the all-gather: each rank's kernel stores every
    finished tile of its column block into its own output AND into the same place of every peer's
    output (peer-mapped symmetric memory, TMA / vector stores over NVLink).  No staging buffer, no
    NCCL call, no re-layout pass; the transfer overlaps the math tile by tile.  Ranks are
    synchronised before the kernel (nobody may still read the previous result) and after it
    (everybody's stores have landed) with the symmetric-memory barrier, which is stream-ordered.
    """

    def __init__(self, m: int, n: int, k: int, group=None, device=None, config=None):
        import ctypes
        self.config = config
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if self.world > 8:
            raise ValueError("at most 8 GPUs (7 peers)")
        self.shard = plan_shard(n, self.world, self.rank)
        self.m, self.n, self.k = m, n, k
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.c_sym, self.handle = symmetric_output(m, n, self.device, self.group)
        self.c_full = self.c_sym.view(1, m, n).permute(1, 2, 0)            # [M, N, 1], row-major
        col_off = self.shard.begin * 2                                      # bytes
        peers = [int(self.handle.buffer_ptrs[r]) + col_off for r in range(self.world) if r != self.rank]
        self.peer_array = (ctypes.c_void_p * max(1, len(peers)))(*peers)
        self.n_peers = len(peers)

    def __call__(self, local_data) -> torch.Tensor:
        from . import _lib
        from .submission import make_problem
        lib = _lib.load()
        c_block = self.c_full[:, self.shard.begin:self.shard.end]          # this rank's columns, row stride N
        problem = make_problem(tuple(local_data[:6]) + (c_block,))
        stream = torch.cuda.current_stream(self.device).cuda_stream
        self.handle.barrier(channel=0)
        _lib.check(lib.nvfp4_gemm_allgather(problem, self.config, self.peer_array, self.n_peers, stream))
        self.handle.barrier(channel=1)
        return self.c_full


class CopyEngineAllGatherGemm:
    """Column-parallel GEMM whose column blocks travel by copy engine.  The rank's GEMM runs row
    panel by row panel straight into its own columns of the full row-major C (symmetric memory);
    as soon as a panel is done, one strided device-to-device copy per peer (cudaMemcpy2DAsync on a
    stream of its own) pushes that panel's column block into the same place of the peer's C while
    the SMs compute the next panel.  No staging, no re-layout, no SM spent on the transfer.
    """

    def __init__(self, m: int, n: int, k: int, group=None, device=None, panels: int = 4):
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.shard = plan_shard(n, self.world, self.rank)
        self.m, self.n, self.k = m, n, k
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.c_sym, self.handle = symmetric_output(m, n, self.device, self.group)
        self.c_full = self.c_sym.view(1, m, n).permute(1, 2, 0)
        self.panels = row_panels(m, panels)
        self.peer_bases = [int(self.handle.buffer_ptrs[r]) for r in range(self.world) if r != self.rank]
        self.copy_streams = [torch.cuda.Stream(device=self.device) for _ in self.peer_bases]

    def __call__(self, local_data) -> torch.Tensor:
        from . import _lib
        from .submission import custom_kernel
        lib = _lib.load()
        a, b, sfa, sfb, sfa_perm, sfb_perm, _ = local_data
        n, nl = self.n, self.shard.n_local
        compute = torch.cuda.current_stream(self.device)
        self.handle.barrier(channel=0)                     # nobody still reads the previous result
        local_base = self.c_sym.data_ptr()
        for (p0, p1) in self.panels:
            rb0, rb1 = p0 // 128, (p1 + 127) // 128
            c_panel = self.c_full[p0:p1, self.shard.begin:self.shard.end]
            custom_kernel((a[p0:p1], b, sfa[p0:p1], sfb, sfa_perm[:, :, rb0:rb1], sfb_perm, c_panel))
            done = torch.cuda.Event()
            done.record(compute)
            off = (p0 * n + self.shard.begin) * 2
            for base, stream in zip(self.peer_bases, self.copy_streams):
                stream.wait_event(done)
                _lib.check(lib.nvfp4_copy_2d(base + off, n * 2, local_base + off, n * 2, nl * 2, p1 - p0, stream.cuda_stream))
        for stream in self.copy_streams:
            ev = torch.cuda.Event()
            ev.record(stream)
            compute.wait_event(ev)
        self.handle.barrier(channel=1)                     # every rank's pushes have landed
        return self.c_full


def plan_block_copies(rank: int, world: int, n_local: int, local_ptr: int, buffer_ptrs, direction: str, block_bytes: int = 0):
    """Source and destination addresses of the copy kernel's column blocks.  A rank's block starts
    ``block_bytes * owner`` bytes into a row (default: fp16 columns, 2 * n_local).  The peer order
    starts with the next rank, so that at any moment the ranks talk to different peers.  Returns
    (peers, src, dst)."""
    bb = block_bytes or n_local * 2
    peers = [(rank + 1 + i) % world for i in range(world - 1)]
    if direction == "pull":      # the blocks the peers own, from their C into mine
        src = [buffer_ptrs[r] + r * bb for r in peers]
        dst = [local_ptr + r * bb for r in peers]
    elif direction == "push":    # the block I own, from my C into theirs
        src = [local_ptr + rank * bb for _ in peers]
        dst = [buffer_ptrs[r] + rank * bb for r in peers]
    else:
        raise ValueError("direction must be 'push' or 'pull'")
    return peers, src, dst


def symmetric_bytes(nbytes: int, device, group):
    """`nbytes` of symmetric memory (uint8) mapped for plain peer accesses; see symmetric_output."""
    import os
    os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "1"
    import torch.distributed._symmetric_memory as symm_mem
    buf = symm_mem.empty((nbytes,), dtype=torch.uint8, device=device)
    handle = symm_mem.rendezvous(buf, group)
    check_no_multicast(handle)
    return buf, handle


class PanelAllGatherGemm:
    """Column-parallel GEMM with the exchange done by this library's copy kernel, row panel by row
    panel, on a second stream while the tensor cores work on the next panel.  Every rank runs its
    GEMM straight into its own columns of the full row-major result (symmetric memory); nothing is
    staged or re-laid-out.

    direction="push": after a panel's GEMM (stream order, no cross-rank wait) the copy kernel
    writes the panel of this rank's column block into every peer's result (stores over NVLink).
    direction="pull": after a panel, a stream-ordered cross-rank barrier tells everyone that this
    panel exists on every rank, and the copy kernel reads the other ranks' blocks of the panel from
    their peer-mapped result (loads over NVLink).

    copy_sms > 0 splits the SMs: the GEMM runs on ``SMs - copy_sms`` persistent CTAs and the copy
    kernel's CTAs are kept on the SMs it leaves free (they would otherwise share the GEMM's SMs and
    slow both down).

    nvfp4_out=True: the GEMM's epilogue re-quantises the result to NVFP4 (packed e2m1 + permuted
    e4m3 scales, the operand form of a following GEMM) and the exchange moves those bytes, 0.5625
    per element instead of 2.  ``result()`` then returns (packed, sf_permuted) views of the full
    matrix instead of the fp16 C.
    """

    def __init__(self, m: int, n: int, k: int, group=None, device=None, panels: int = 4, copy_ctas: int = 0, direction: str = "push",
                 copy_sms: int = 0, nvfp4_out: bool = False):
        import ctypes
        if direction not in ("push", "pull"):
            raise ValueError("direction must be 'push' or 'pull'")
        self.direction = direction
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if self.world > 8:
            raise ValueError("at most 8 GPUs (7 peers)")
        self.shard = plan_shard(n, self.world, self.rank)
        self.m, self.n, self.k = m, n, k
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.panels = row_panels(m, panels)
        self.copy_stream = torch.cuda.Stream(device=self.device)
        self.nvfp4_out = nvfp4_out
        sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.copy_sms = max(0, min(int(copy_sms), sms - 2))
        self.gemm_grid = ((sms - self.copy_sms) // 2) * 2 if self.copy_sms else 0
        self.copy_ctas = self.copy_sms * 8 if self.copy_sms else copy_ctas
        nl = self.shard.n_local
        if not nvfp4_out:
            self.c_sym, self.handle = symmetric_output(m, n, self.device, self.group)
            self.c_full = self.c_sym.view(1, m, n).permute(1, 2, 0)
            ptrs = [int(p) for p in self.handle.buffer_ptrs]
            # (address lists of one copy launch per panel: geometry in fp16 elements)
            self.copies = [self._copy_plan(self.c_sym.data_ptr(), ptrs, nl * 2, nl, n, rows_scale=1)]
        else:
            if m % 128 or nl % 64:
                raise ValueError("the NVFP4 exchange needs m % 128 == 0 and (n / world) % 64 == 0")
            self.packed_bytes = m * (n // 2)
            self.perm_bytes = (m // 128) * (n // 64) * 512
            self.buf, self.handle = symmetric_bytes(self.packed_bytes + self.perm_bytes, self.device, self.group)
            ptrs = [int(p) for p in self.handle.buffer_ptrs]
            base = self.buf.data_ptr()
            # a byte matrix is moved by counting two bytes as one 16-bit element
            self.copies = [
                self._copy_plan(base, ptrs, nl // 2, nl // 4, n // 4, rows_scale=1),                                   # packed rows
                self._copy_plan(base + self.packed_bytes, [p + self.packed_bytes for p in ptrs], (nl // 64) * 512,
                                (nl // 64) * 256, (n // 64) * 256, rows_scale=128),                                    # scale atoms, per 128 rows
            ]

    def _copy_plan(self, local_ptr, buffer_ptrs, block_bytes, n_local_el, row_stride_el, rows_scale):
        import ctypes
        peers, src, dst = plan_block_copies(self.rank, self.world, 0, local_ptr, buffer_ptrs, self.direction, block_bytes=block_bytes)
        return dict(src=(ctypes.c_void_p * len(peers))(*src), dst=(ctypes.c_void_p * len(peers))(*dst), n=len(peers),
                    n_local=n_local_el, row_stride=row_stride_el, rows_scale=rows_scale)

    def result(self):
        if not self.nvfp4_out:
            return self.c_full
        from .inputs import FP4_DTYPE, SF_DTYPE
        packed = self.buf[:self.packed_bytes].view(1, self.m, self.n // 2).permute(1, 2, 0).view(FP4_DTYPE)
        perm = self.buf[self.packed_bytes:].view(1, self.m // 128, self.n // 64, 32, 4, 4).permute(3, 4, 1, 5, 2, 0).view(SF_DTYPE)
        return packed, perm

    def _gemm_panel(self, lib, local_data, p0, p1, stream):
        from . import _lib
        from .submission import make_problem
        a, b, sfa, sfb, sfa_perm, sfb_perm, _ = local_data
        rb0, rb1 = p0 // 128, (p1 + 127) // 128
        cfg = _lib.GemmConfig(0, 0, self.gemm_grid, 0, 0, 0)
        if not self.nvfp4_out:
            c_panel = self.c_full[p0:p1, self.shard.begin:self.shard.end]
            problem = make_problem((a[p0:p1], b, sfa[p0:p1], sfb, sfa_perm[:, :, rb0:rb1], sfb_perm, c_panel))
            _lib.check(lib.nvfp4_gemm(problem, cfg, stream))
            return
        problem = make_problem((a[p0:p1], b, sfa[p0:p1], sfb, sfa_perm[:, :, rb0:rb1], sfb_perm, None))
        n, nl = self.n, self.shard.n_local
        epi = _lib.Epilogue()
        epi.output = _lib.OUT_NVFP4
        base = self.buf.data_ptr()
        epi.out_packed = base + p0 * (n // 2) + self.rank * (nl // 2)
        epi.out_packed_row_stride = n // 2
        epi.out_sf_perm = base + self.packed_bytes + rb0 * (n // 64) * 512 + self.rank * (nl // 64) * 512
        epi.out_sf_perm_block_stride = (n // 64) * 512
        _lib.check(lib.nvfp4_gemm_epilogue(problem, cfg, epi, stream))

    def __call__(self, local_data):
        from . import _lib
        lib = _lib.load()
        compute = torch.cuda.current_stream(self.device)
        self.handle.barrier(channel=0)                     # nobody still reads the previous result
        for idx, (p0, p1) in enumerate(self.panels):
            self._gemm_panel(lib, local_data, p0, p1, compute.cuda_stream)
            if self.direction == "pull":
                self.handle.barrier(channel=1 + idx % 2)   # this panel now exists on every rank
            ready = torch.cuda.Event()
            ready.record(compute)
            self.copy_stream.wait_event(ready)
            for cp in self.copies:
                _lib.check(lib.nvfp4_copy_column_blocks(cp["dst"], cp["src"], cp["n"], p0 // cp["rows_scale"], (p1 - p0) // cp["rows_scale"],
                                                        cp["n_local"], cp["row_stride"], self.copy_ctas, 1 if self.copy_sms else 0,
                                                        self.copy_stream.cuda_stream))
        done = torch.cuda.Event()
        done.record(self.copy_stream)
        compute.wait_event(done)
        if self.direction == "push":
            self.handle.barrier(channel=1)                 # every rank's blocks have landed here
        return self.result()


def best_allgather_mode(world: int) -> str:
    """Measured on B200 / NVSwitch for the 8192 x 28672 x 8192 job: with two GPUs the GEMM dominates
    and the epilogue's peer stores hide best; from four GPUs on the exchange dominates and the copy
    kernel pushing finished row panels keeps the links fuller than the epilogue does."""
    return "fused" if world <= 2 else "push"
