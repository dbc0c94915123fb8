"""Host-side logic of the column-parallel GEMM on two CPU ranks (gloo): sharding, panel
pipeline, all-gather and the column-block re-layout, with the oracle standing in for the GPU
kernel (the product path has no such stand-in: its defaults are the CUDA library)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, m, n, k, panels, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from nvfp4_gemm_b200.inputs import generate_input
    from nvfp4_gemm_b200.multi_gpu import ColumnParallelGemm, plan_shard, shard_inputs
    from oracle import nvfp4_oracle as O

    full = generate_input(m, n, k, 1, 1111, device="cpu")
    shard = plan_shard(n, world, rank)
    local = shard_inputs(full, shard)
    assert local[1].shape[0] == n // world and local[5].shape[2] == n // world // 128

    def gemm_fn(panel):
        a, b, sfa, sfb = O.tensors_to_numpy(panel)
        # read the PERMUTED scales, as the GPU kernel does: checks that their slicing is right
        pa = torch.as_strided(panel[4].view(torch.uint8), (32, 4, panel[4].shape[2], 4, panel[4].shape[4]),
                              panel[4].stride()[:5]).permute(2, 4, 0, 1, 3).contiguous().numpy().reshape(-1)
        pb = torch.as_strided(panel[5].view(torch.uint8), (32, 4, panel[5].shape[2], 4, panel[5].shape[4]),
                              panel[5].stride()[:5]).permute(2, 4, 0, 1, 3).contiguous().numpy().reshape(-1)
        c = O.ref_gemm_from_permuted(a, b, pa, pb)
        panel[6].copy_(torch.from_numpy(c))

    def interleave_fn(src, dst, rows, n_local, blocks, dst_row_stride):
        assert src.shape == (blocks, rows, n_local) and dst_row_stride == n
        dst[:, :, 0] = src.permute(1, 0, 2).reshape(rows, blocks * n_local)

    plan = ColumnParallelGemm(m, n, k, device="cpu", panels=panels, gemm_fn=gemm_fn, interleave_fn=interleave_fn)
    c_full = torch.zeros((1, m, n), dtype=torch.float16).permute(1, 2, 0)
    plan(local, c_full)
    a, b, sfa, sfb = O.tensors_to_numpy(full)
    exp = O.ref_gemm(a, b, sfa, sfb)
    ok = np.array_equal(c_full.numpy().view(np.uint16), exp.view(np.uint16))
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
        f.write("ok" if ok else "mismatch")
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("m,n,k,panels", [(512, 512, 256, 2), (300, 256, 512, 4)])
def test_two_rank_column_parallel_on_cpu(tmp_path, m, n, k, panels):
    world = 2
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, m, n, k, panels, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert (tmp_path / f"rank{r}.txt").read_text() == "ok"


def test_shard_plan_and_panels():
    from nvfp4_gemm_b200.multi_gpu import plan_shard, row_panels
    s = plan_shard(28672, 8, 3)
    assert (s.n_local, s.begin, s.end) == (3584, 10752, 14336)
    with pytest.raises(ValueError):
        plan_shard(1000, 8, 0)
    with pytest.raises(ValueError):
        plan_shard(1024, 2, 2)
    assert row_panels(8192, 4) == [(0, 2048), (2048, 4096), (4096, 6144), (6144, 8192)]
    assert row_panels(300, 4) == [(0, 256), (256, 300)]
    assert row_panels(100, 4) == [(0, 100)]
    cover = row_panels(4097, 3)
    assert cover[0][0] == 0 and cover[-1][1] == 4097 and all(a[1] == b[0] for a, b in zip(cover, cover[1:]))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_block_copy_plan_covers_every_foreign_block_once(world):
    """The copy kernel's address lists: pull reads each peer's own block into the same place of the
    local output, push writes the local block into the same place of each peer's output; at a given
    position of the list every rank addresses a different peer."""
    from nvfp4_gemm_b200.multi_gpu import best_allgather_mode, plan_block_copies
    n_local = 256
    bases = [0x10000000 * (r + 1) for r in range(world)]
    order = []
    for rank in range(world):
        peers, src, dst = plan_block_copies(rank, world, n_local, bases[rank], bases, "pull")
        assert sorted(peers) == [r for r in range(world) if r != rank]
        for r, s, d in zip(peers, src, dst):
            assert s == bases[r] + r * n_local * 2 and d == bases[rank] + r * n_local * 2
        peers2, src2, dst2 = plan_block_copies(rank, world, n_local, bases[rank], bases, "push")
        assert peers2 == peers
        for r, s, d in zip(peers2, src2, dst2):
            assert s == bases[rank] + rank * n_local * 2 and d == bases[r] + rank * n_local * 2
        order.append(peers)
    for pos in range(world - 1):
        assert sorted(o[pos] for o in order) == list(range(world))
    with pytest.raises(ValueError):
        plan_block_copies(0, world, n_local, bases[0], bases, "sideways")
    assert best_allgather_mode(2) == "fused" and best_allgather_mode(8) == "push"


def test_multicast_binding_is_refused():
    """The symmetric output must be mapped for plain peer accesses only; a rendezvous handle that
    reports a multicast address is an error (fake handles: no GPU needed)."""
    from types import SimpleNamespace
    from nvfp4_gemm_b200.multi_gpu import check_no_multicast
    check_no_multicast(SimpleNamespace(multicast_ptr=0))
    check_no_multicast(SimpleNamespace())                      # torch builds without the attribute
    with pytest.raises(RuntimeError, match="multicast"):
        check_no_multicast(SimpleNamespace(multicast_ptr=0x7F0000000000))


def test_block_copy_plan_for_byte_blocks():
    """The NVFP4 exchange moves byte matrices (packed values, scale atoms): a rank's block then
    starts block_bytes * owner into a row, whatever n_local says."""
    from nvfp4_gemm_b200.multi_gpu import plan_block_copies
    world, bb = 4, 1792
    bases = [0x1000_0000 * (r + 1) for r in range(world)]
    for rank in range(world):
        peers, src, dst = plan_block_copies(rank, world, 0, bases[rank], bases, "push", block_bytes=bb)
        assert sorted(peers) == [r for r in range(world) if r != rank]
        assert all(s == bases[rank] + rank * bb for s in src)
        assert dst == [bases[r] + rank * bb for r in peers]
        peers, src, dst = plan_block_copies(rank, world, 0, bases[rank], bases, "pull", block_bytes=bb)
        assert src == [bases[r] + r * bb for r in peers] and dst == [bases[rank] + r * bb for r in peers]
