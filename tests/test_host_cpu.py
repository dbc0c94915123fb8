"""Host-side logic that needs no GPU: the C ABI loads and exports what the header declares,
argument validation, the work partition, and the tuple -> problem translation."""
import ctypes
import os
import re

import pytest
import torch

from nvfp4_gemm_b200 import _lib
from nvfp4_gemm_b200.inputs import generate_input
from nvfp4_gemm_b200.submission import custom_kernel, make_problem

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(lib):
    header = open(os.path.join(ROOT, "include", "nvfp4_b200.h")).read()
    declared = set(re.findall(r"\b(nvfp4_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found in the header"
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/nvfp4_b200.h but not exported"
    assert set(_lib.EXPORTED_SYMBOLS) <= declared
    assert b"sm_100a" in lib.nvfp4_version()


def test_make_problem_strides():
    data = generate_input(256, 384, 512, 2, 1, device="cpu")
    p = make_problem(data)
    assert (p.m, p.n, p.k, p.l) == (256, 384, 512, 2)
    assert p.a_row_stride == 256 and p.a_batch_stride == 256 * 256
    assert p.b_row_stride == 256 and p.b_batch_stride == 384 * 256
    assert p.sfa_row_stride == 32 and p.sfa_batch_stride == 256 * 32
    assert p.sfa_perm_batch_stride == 2 * 8 * 512 and p.sfb_perm_batch_stride == 3 * 8 * 512
    assert p.c_row_stride == 384 and p.c_batch_stride == 256 * 384
    gv = make_problem(generate_input(64, 1, 256, 3, 1, device="cpu"))
    assert gv.n == 1 and gv.c_row_stride == 1 and gv.c_batch_stride == 64 and gv.b_batch_stride == 128


def test_custom_kernel_refuses_cpu_tensors(lib):
    with pytest.raises(ValueError, match="no CPU fallback"):
        custom_kernel(generate_input(128, 128, 256, 1, 1, device="cpu"))


def _problem(**over):
    data = generate_input(128, 256, 512, 1, 1, device="cpu")
    p = make_problem(data)
    for k, v in over.items():
        setattr(p, k, v)
    return p, data


@pytest.mark.parametrize("over,msg", [
    (dict(k=300), "multiple of 256"),
    (dict(n=200), "multiple of 128"),
    (dict(m=0), "positive"),
    (dict(a=None), "must not be NULL"),
    (dict(sfa_perm=None), "permuted scale"),
    (dict(a_row_stride=250), "row strides"),
    (dict(c_row_stride=257), "c_row_stride"),
])
def test_gemm_rejects_bad_arguments_before_touching_the_gpu(lib, over, msg):
    p, _keep = _problem(**over)
    rc = lib.nvfp4_gemm(p, None, None)
    assert rc == _lib.NVFP4_ERR_INVALID_ARGUMENT
    assert msg in lib.nvfp4_last_error().decode()


def test_gemm_rejects_misaligned_pointer(lib):
    p, _keep = _problem()
    p.b = p.b + 8
    assert lib.nvfp4_gemm(p, None, None) == _lib.NVFP4_ERR_INVALID_ARGUMENT
    cfg = _lib.GemmConfig(64, 0, 0, 0)
    p, _keep = _problem()
    assert lib.nvfp4_gemm(p, cfg, None) == _lib.NVFP4_ERR_INVALID_ARGUMENT


def test_gemv_rejects_bad_arguments(lib):
    data = generate_input(64, 1, 256, 1, 1, device="cpu")
    p = make_problem(data)
    p.k = 100
    assert lib.nvfp4_gemv(p, None) == _lib.NVFP4_ERR_INVALID_ARGUMENT
    p = make_problem(data)
    p.n = 2
    assert lib.nvfp4_gemv(p, None) == _lib.NVFP4_ERR_INVALID_ARGUMENT
    p = make_problem(data)
    p.sfa = None
    assert lib.nvfp4_gemv(p, None) == _lib.NVFP4_ERR_INVALID_ARGUMENT


@pytest.mark.parametrize("total,grid,kt", [(3584, 148, 64), (1792, 148, 64), (896 * 28, 148, 28), (7, 7, 1), (100, 148, 4), (229376, 148, 32)])
def test_work_partition_covers_every_unit_once_and_is_balanced(lib, total, grid, kt):
    grid = min(grid, total)
    b, e, slot = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    prev_end = 0
    sizes, slots = [], set()
    for cta in range(grid):
        assert lib.nvfp4_plan_units(total, grid, cta, ctypes.byref(b), ctypes.byref(e), ctypes.byref(slot), kt) == 0
        assert b.value == prev_end and e.value >= b.value
        prev_end = e.value
        sizes.append(e.value - b.value)
        # a worker's first segment uses its "head" slot when it starts inside a tile, else its "tail" slot
        assert slot.value == 2 * cta + (0 if b.value % kt else 1)
        slots.add(slot.value)
    assert prev_end == total
    assert max(sizes) - min(sizes) <= 1            # stream-K balance
    assert len(slots) == grid                      # no two workers share a partial-tile slot
    assert lib.nvfp4_plan_units(total, grid, grid, ctypes.byref(b), ctypes.byref(e), None, kt) == _lib.NVFP4_ERR_INVALID_ARGUMENT


@pytest.mark.parametrize("total,grid,kt", [(448 * 28, 74, 28), (3584 * 32, 74, 32), (56 * 64, 148, 64), (7, 7, 1), (100, 148, 4), (2 * 28, 148, 28), (5 * 8, 3, 8)])
def test_segment_order_partitions_a_workers_range_and_ends_on_a_whole_tile(lib, total, grid, kt):
    grid = min(grid, total)
    b, e, sb, se = ctypes.c_int(), ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    covered = [0] * total
    for cta in range(grid):
        assert lib.nvfp4_plan_units(total, grid, cta, ctypes.byref(b), ctypes.byref(e), None, kt) == 0
        segs = []
        for i in range(total // kt + 4):
            assert lib.nvfp4_plan_segment(total, grid, cta, kt, i, ctypes.byref(sb), ctypes.byref(se)) == 0
            if sb.value < 0:
                break
            segs.append((sb.value, se.value))
        else:
            raise AssertionError("the segment sequence does not end")
        assert sorted(segs)[0][0] == b.value and sorted(segs)[-1][1] == e.value
        for u0, u1 in segs:
            assert u0 < u1 and u0 // kt == (u1 - 1) // kt                     # inside one tile
            for u in range(u0, u1):
                covered[u] += 1
        whole = [sg for sg in segs if sg[1] - sg[0] == kt]
        assert whole == sorted(whole)
        if b.value % kt and segs:                                             # published partial: first of all
            assert segs[0][0] == b.value
        if e.value % kt and (e.value // kt) * kt >= b.value + ((-b.value) % kt):   # finished partial ...
            tail = ((e.value // kt) * kt, e.value)
            if tail[0] >= b.value:
                pos = segs.index(tail)
                assert pos == (len(segs) - 2 if whole else len(segs) - 1)     # ... last but one, before the last whole tile
    assert covered == [1] * total
    assert lib.nvfp4_plan_segment(total, grid, grid, kt, 0, ctypes.byref(sb), ctypes.byref(se)) == _lib.NVFP4_ERR_INVALID_ARGUMENT


@pytest.mark.parametrize("tiles,k_tiles,max_workers,exp_workers,exp_whole", [
    (448, 28, 74, 74, 0),        # 4096 x 7168 x 7168 on pairs: 6.05 tiles per worker, even split
    (3584, 32, 74, 74, 0),       # 8192 x 28672 x 8192
    (162, 28, 74, 74, 0),        # 2304 x 4608 x 7168: 2.2 tiles per worker, the summing hides behind whole tiles
    (48, 16, 74, 48, 1),         # 768 x 4096 x 4096: fewer tiles than pairs, one whole tile each
    (112, 16, 74, 56, 1),        # 1024 x 7168 x 4096: two waves, on the fewest workers that need two
    (56, 8, 148, 56, 1),         # 128 x 7168 x 2048 on single CTAs
    (1, 64, 148, 1, 1),
])
def test_work_split_choice(lib, tiles, k_tiles, max_workers, exp_workers, exp_whole):
    w, whole = ctypes.c_int(), ctypes.c_int()
    assert lib.nvfp4_plan_work_split(tiles, k_tiles, max_workers, ctypes.byref(w), ctypes.byref(whole)) == 0
    assert (w.value, whole.value) == (exp_workers, exp_whole)
    if whole.value:                                        # no more waves than the full device would need
        waves = -(-tiles // min(tiles, max_workers))
        assert -(-tiles // w.value) == waves
    assert lib.nvfp4_plan_work_split(0, k_tiles, max_workers, ctypes.byref(w), ctypes.byref(whole)) == _lib.NVFP4_ERR_INVALID_ARGUMENT


@pytest.mark.parametrize("m,n,k,exp", [
    (4096, 7168, 7168, (2, 256)), (8192, 28672, 8192, (2, 256)), (2304, 4608, 7168, (2, 256)),      # large: pairs
    (512, 7168, 2048, (2, 256)), (768, 4096, 4096, (2, 256)), (1024, 7168, 4096, (2, 256)), (384, 7168, 2304, (2, 256)),
    (1536, 4096, 4096, (2, 256)),
    (1024, 4096, 1024, (1, 128)), (640, 7168, 7168, (1, 128)), (512, 1536, 7168, (1, 128)), (256, 7168, 256, (1, 128)),
    (512, 4096, 512, (1, 128)), (256, 7168, 2048, (1, 128)),                                          # small / short K: single CTAs
    (128, 7168, 2048, (1, 128)), (256, 384, 1024, (1, 128)),                                          # one row block; N not a multiple of 256
])
def test_tile_shape_choice_on_a_148_sm_device(lib, m, n, k, exp):
    """The choices measured on a B200 (each row was timed with both tiles; the faster one is expected)."""
    cg, bn = ctypes.c_int(), ctypes.c_int()
    assert lib.nvfp4_plan_tile_shape(m, n, k, 1, 148, ctypes.byref(cg), ctypes.byref(bn)) == 0
    assert (cg.value, bn.value) == exp
    assert lib.nvfp4_plan_tile_shape(m, n + 1, k, 1, 148, ctypes.byref(cg), ctypes.byref(bn)) == _lib.NVFP4_ERR_INVALID_ARGUMENT


def test_bench_roofline_arithmetic_matches_the_stated_work():
    """Algorithmic flops / bytes per launch that bench.py divides by the measured time: the
    figures of the task's configurations (2*M*N*K*L and the packed operand, scale and output bytes)."""
    import importlib.util
    import os
    spec = importlib.util.spec_from_file_location("bench", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    w = bench.WORKLOADS
    assert bench.algorithmic_flops(w["c1"]) == 30_064_771_072 and bench.algorithmic_bytes(w["c1"]) == 69_074_944
    assert bench.algorithmic_flops(w["c2"]) == 939_524_096 and bench.algorithmic_bytes(w["c2"]) == 264_335_360
    assert bench.algorithmic_flops(w["c3"]) == 420_906_795_008 and bench.algorithmic_bytes(w["c3"]) == 104_136_704
    assert bench.algorithmic_flops(w["c4"]) == 3_848_290_697_216
    for key, shape in bench.LEADERBOARD.items():
        assert shape["sol_us"] > 0
        if "m" in shape:
            assert shape["k"] % 64 == 0 and (shape["n"] == 1 or shape["n"] % 128 == 0)


def test_problem_cache_key_covers_strides_and_none_scales():
    """Same storage seen through two stride layouts gives two distinct problem structs, and a
    GEMV-only call may leave the permuted scale tensors out."""
    import torch
    from nvfp4_gemm_b200 import submission as S
    from nvfp4_gemm_b200.inputs import generate_input
    data = generate_input(64, 1, 512, 1, 3, device="cpu")
    p = S.make_problem(data[:4] + (None, None, data[6]))
    assert p.sfa_perm is None and p.sfb_perm is None and p.n == 1
    store = torch.zeros(64 * 512, dtype=torch.uint8)
    v1 = torch.as_strided(store, (32, 256, 1), (256, 1, 32 * 256))
    v2 = torch.as_strided(store, (32, 256, 1), (512, 1, 32 * 512))
    assert v1.data_ptr() == v2.data_ptr() and S._layout_key(v1) != S._layout_key(v2)
    assert S._layout_key(None) == (0, (), ())


@pytest.mark.parametrize("raster", [0, 1, 8, 16])
@pytest.mark.parametrize("tiles_m,tiles_n,batches,k_tiles,workers", [(16, 28, 1, 28, 74), (32, 112, 1, 32, 74), (9, 18, 1, 28, 74),
                                                                    (3, 5, 2, 4, 7), (1, 3, 1, 16, 148), (17, 4, 3, 2, 10), (2, 2, 1, 8, 4)])
def test_tile_order_visits_every_output_tile_once(lib, tiles_m, tiles_n, batches, k_tiles, workers, raster):
    import ctypes
    tiles = tiles_m * tiles_n * batches
    seen = set()
    b, r, c = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    for t in range(tiles):
        assert lib.nvfp4_plan_tile(tiles * k_tiles, workers, k_tiles, tiles_m, tiles_n, raster, t, ctypes.byref(b), ctypes.byref(r), ctypes.byref(c)) == 0
        assert 0 <= b.value < batches and 0 <= r.value < tiles_m and 0 <= c.value < tiles_n
        seen.add((b.value, r.value, c.value))
    assert len(seen) == tiles
    assert lib.nvfp4_plan_tile(tiles * k_tiles, workers, k_tiles, tiles_m, tiles_n, raster, tiles, ctypes.byref(b), ctypes.byref(r), ctypes.byref(c)) != 0
