"""CPU checks of the boundary: the C-ABI library loads, exports every symbol the header declares,
refuses non-CUDA tensors loudly, and the work splitter's arithmetic holds its invariants."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

from void_b200 import _lib
import void_b200 as void

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "void_b200.h")).read()
    return sorted(set(re.findall(r"VOID_API[^;(]*?\b(void_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(_lib.lib_path()) if os.path.exists(_lib.lib_path()) else _lib.load()
    names = declared_symbols()
    assert len(names) >= 18
    for name in names:
        assert hasattr(lib, name), name
    assert sorted(_lib.EXPORTED_SYMBOLS) == names  # the ctypes table binds exactly the header


def test_library_loads_and_reports_errors():
    lib = _lib.load()
    assert lib.void_b200_abi_version() == _lib.ABI_VERSION == 5
    assert lib.void_strerror(0) == b"ok"
    assert b"alignment" in lib.void_strerror(-2)
    with pytest.raises(_lib.VoidB200Error):
        _lib.check(-3, "x")


def test_ctypes_mirror_matches_the_c_struct_layout(tmp_path):
    # the header compiled as plain C: size and field offsets of void_spmm_args must be what the ctypes mirror assumes
    import shutil
    import subprocess
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    fields = [name for name, _ in _lib.SpmmArgs._fields_]
    src = tmp_path / "layout.c"
    src.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "void_b200.h"\nint main(void) {\n'
                   '  printf("%zu\\n", sizeof(void_spmm_args));\n'
                   + "".join('  printf("%%zu\\n", offsetof(void_spmm_args, %s));\n' % f for f in fields)
                   + "  return 0;\n}\n")
    exe = tmp_path / "layout"
    subprocess.run([gcc, "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)],
                   check=True)
    out = [int(x) for x in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()]
    assert out[0] == ctypes.sizeof(_lib.SpmmArgs)
    assert out[1:] == [getattr(_lib.SpmmArgs, f).offset for f in fields]


def test_no_cpu_fallback():
    import scipy.sparse as sp
    a = void.csr_to_void(sp.random(64, 64, density=0.2, format="csr", dtype=np.float32, random_state=1))
    assert a.values.device.type == "cpu"
    with pytest.raises(_lib.VoidB200Error, match="no CPU path"):
        a.get_row_block_info()
    with pytest.raises(_lib.VoidB200Error, match="no CPU path"):
        void.quantize_void_tensor(a)
    with pytest.raises(_lib.VoidB200Error, match="no CPU path"):
        void.void_tensor_to_fp8(a)


def test_floating_point_and_training_operators_refuse_cpu_tensors():
    import scipy.sparse as sp
    a = void.csr_to_void(sp.random(64, 96, density=0.2, format="csr", dtype=np.float32, random_state=2))
    b = torch.randn(96, 8)
    for call in (lambda: void.void_spmm(a, b), lambda: void.void_spmv(a, b[:, 0]), lambda: void.void_spmm_gelu(a, b),
                 lambda: void.void_spmm_stream_k(a, b), lambda: void.dense_to_void(torch.randn(64, 64)),
                 lambda: void.spmm_tile_grad(a, torch.randn(64, 8), b),
                 lambda: void.fused_sparse_mlp(torch.randn(4, 96), a, a)):
        with pytest.raises(_lib.VoidB200Error, match="no CPU path"):
            call()


def test_tile_grad_items_cover_every_tile_once():
    # groups of at most four consecutive packed tiles, never across a tile row (host-side index arithmetic)
    from void_b200.autograd import tile_grad_items
    row_ptr = torch.tensor([0, 0, 5, 5, 6, 14, 14, 17], dtype=torch.int32)
    items = tile_grad_items(row_ptr).numpy()
    assert items.dtype == np.int32 and items.shape[1] == 4
    assert items[:, :3].tolist() == [[1, 0, 4], [1, 4, 1], [3, 5, 1], [4, 6, 4], [4, 10, 4], [6, 14, 3]]
    covered = np.concatenate([np.arange(t0, t0 + n) for _, t0, n, _ in items])
    assert covered.tolist() == list(range(17))
    assert tile_grad_items(torch.zeros(4, dtype=torch.int32)).shape == (0, 4)


def test_product_kind_follows_the_operand_types():
    from void_b200.ops import product_kind
    import scipy.sparse as sp
    a = void.csr_to_void(sp.random(64, 64, density=0.2, format="csr", dtype=np.float32, random_state=3))
    assert product_kind(a, torch.zeros(64, 4)) == _lib.KIND_TF32
    assert product_kind(a.half(), torch.zeros(64, 4, dtype=torch.float16)) == _lib.KIND_F16
    assert product_kind(a.bfloat16(), torch.zeros(64, 4, dtype=torch.bfloat16)) == _lib.KIND_BF16
    assert product_kind(a.half(), torch.zeros(64, 4)) == _lib.KIND_TF32          # mixed: through fp32, like the reference's casts
    with pytest.raises(_lib.VoidB200Error):
        product_kind(a, torch.zeros(64, 4, dtype=torch.int8))


def test_package_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "void_b200")
    for fn in os.listdir(pkg):
        if fn.endswith(".py"):
            src = open(os.path.join(pkg, fn)).read()
            assert "oracle" not in src, fn


def test_streamk_target_matches_reference_formula():
    lib = _lib.load()
    for nnz, req, mw in [(7976, -1, 16), (100, -1, 16), (5000, 64, 16), (5000, 300, 4), (3, 7, 16), (1609, -1, 16)]:
        n_workers = req if req > 0 else min(nnz, 1024)
        assert lib.void_streamk_target(nnz, req, mw) == min((nnz + n_workers - 1) // n_workers, mw)
    assert lib.void_streamk_target(0, -1, 16) == 0


def _plan(row_ptr, n_chunks, n_cta, mode, T, row_cost=1):
    lib = _lib.load()
    nbr = len(row_ptr) - 1
    nnz = int(row_ptr[-1])
    cap = lib.void_plan_capacity(nnz, nbr, n_chunks, n_cta, mode, T)
    segs = np.zeros((cap, 8), np.int32)
    cptr = np.zeros(n_cta + 1, np.int32)
    counts = np.zeros(4, np.int32)
    woff = None
    if mode == 2:
        cnt = np.diff(row_ptr)
        woff = np.concatenate([[0], np.cumsum((cnt + T - 1) // T)]).astype(np.int32)
    st = lib.void_plan_segments_host(row_ptr.ctypes.data, nbr, n_chunks, n_cta, mode, T, row_cost,
                                     None if woff is None else woff.ctypes.data, segs.ctypes.data, cap,
                                     cptr.ctypes.data, counts.ctypes.data)
    assert st == 0 and counts[3] == 0
    return segs[:counts[0]], cptr, counts


def _check_plan(row_ptr, n_chunks, n_cta, mode, T, row_cost=1):
    segs, cptr, counts = _plan(row_ptr, n_chunks, n_cta, mode, T, row_cost)
    nbr = len(row_ptr) - 1
    assert cptr[0] == 0 and cptr[-1] == len(segs) and (np.diff(cptr) >= 0).all()
    rows = {}
    for row, ch, t0, t1, nseg, slot0, idx, ctr in segs:
        assert row_ptr[row] <= t0 <= t1 <= row_ptr[row + 1]
        rows.setdefault((ch, row), []).append((t0, t1, nseg, slot0, idx, ctr))
    assert len(rows) == nbr * n_chunks            # every (chunk, tile row) is written by someone
    slots, ctrs = set(), set()
    for (ch, row), ps in rows.items():
        ps.sort()
        assert ps[0][0] == row_ptr[row] and ps[-1][1] == row_ptr[row + 1]
        assert all(a[1] == b[0] for a, b in zip(ps[:-1], ps[1:]))   # tiles covered exactly once
        assert all(p[2] == len(ps) for p in ps)
        if len(ps) > 1:
            assert mode > 0
            assert [p[4] for p in ps] == list(range(len(ps)))
            assert len({p[3] for p in ps}) == 1 and len({p[5] for p in ps}) == 1
            for p in ps:
                assert p[1] > p[0] and p[3] + p[4] < counts[1] and (p[3] + p[4]) not in slots
                slots.add(p[3] + p[4])
            assert ps[0][5] < counts[2] and ps[0][5] not in ctrs
            ctrs.add(ps[0][5])
            if mode == 2:
                assert all(p[1] - p[0] <= T for p in ps)
    return segs, cptr


def test_plan_invariants_random():
    rng = np.random.default_rng(0)
    for trial in range(120):
        nbr = int(rng.integers(1, 150))
        kind = trial % 3
        if kind == 0:
            cnt = rng.integers(0, 20, nbr)
        elif kind == 1:
            cnt = np.minimum(rng.zipf(1.5, nbr), 512)
        else:
            cnt = (rng.random(nbr) < 0.3) * rng.integers(0, 300, nbr)
        row_ptr = np.concatenate([[0], np.cumsum(cnt)]).astype(np.int32)
        if row_ptr[-1] == 0:
            continue
        for mode in (0, 1, 2):
            _check_plan(row_ptr, int(rng.integers(1, 4)), int(rng.integers(1, 300)), mode, int(rng.integers(1, 17)),
                        int(rng.integers(1, 12)))


def test_plan_splits_heavy_rows_only_when_asked():
    cnt = np.full(64, 4)
    cnt[10] = 400                                  # one row far heavier than a CTA's share
    row_ptr = np.concatenate([[0], np.cumsum(cnt)]).astype(np.int32)
    segs0, _ = _check_plan(row_ptr, 1, 32, 0, 8)
    assert (segs0[:, 4] == 1).all()
    segs1, cptr1 = _check_plan(row_ptr, 1, 32, 1, 8)
    heavy = segs1[segs1[:, 0] == 10]
    assert len(heavy) > 4 and (heavy[:, 4] == len(heavy)).all()
    assert (segs1[segs1[:, 0] != 10][:, 4] == 1).all()
    work = np.array([sum(s[3] - s[2] for s in segs1[cptr1[k]:cptr1[k + 1]]) for k in range(32)])
    assert work.max() <= 3 * work.mean()


def test_row_range_matches_reference_formula():
    from void_b200.distributed import row_range
    for nbr, world in [(2048, 8), (128, 3), (5, 8), (96, 4)]:
        rpr = (nbr + world - 1) // world
        got = [row_range(nbr, world, r) for r in range(world)]
        for r, (s, e) in enumerate(got):
            assert s == min(r * rpr, nbr) and e == min(s + rpr, nbr)
        assert got[0][0] == 0 and max(e for _, e in got) == nbr
