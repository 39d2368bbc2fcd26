"""GPU parity of the training side: VOIDSpMMFunction / VOIDSpMM / SparseLinear against gradients produced by
the reference's own autograd function and against torch's dense autograd.  Bars as in the reference's
tests/test_backward.py (:81, :103: rtol = atol = 1e-2 for TF32), tightened where the arithmetic allows."""
import numpy as np
import pytest
import torch

import void_b200 as void
from void_b200 import workloads
from conftest import coo_to_csr, load_golden, rel_err
from oracle import void_oracle as vo

pytestmark = pytest.mark.gpu


def _np(t):
    return t.detach().float().cpu().numpy()


def test_gradients_vs_reference_autograd_output():
    g = load_golden("backward_small.npz")
    a = void.csr_to_void(coo_to_csr(g), tile_size=32, device="cuda")
    assert np.array_equal(_np(a.block_rows), g["block_rows"]) and np.array_equal(_np(a.block_cols), g["block_cols"])
    vals = a.values.clone().requires_grad_(True)
    b = torch.from_numpy(g["b"]).cuda().requires_grad_(True)
    c = void.VOIDSpMMFunction.apply(vals, a.block_rows, a.block_cols, a.shape, a.tile_size, a.n_blocks, b)
    assert rel_err(_np(c), g["c"]) < 1e-3
    c.backward(torch.from_numpy(g["grad_c"]).cuda())
    assert vals.grad.shape == a.values.shape and rel_err(_np(vals.grad), g["grad_values"]) < 1e-3
    assert b.grad.shape == (150, 72) and rel_err(_np(b.grad), g["grad_b"]) < 1e-3
    void.check_device_status()


def test_tile_grad_exact_on_small_integers():
    # integer operands below 2^10 are exact in TF32 / fp16 / bf16 and the sums stay exact in fp32
    mask = workloads.uniform_mask(9, 7, 0.4, seed=3)
    mask[2] = False
    gen = torch.Generator().manual_seed(1)
    tiles = torch.randint(-3, 4, (int(mask.sum()), 32, 32), generator=gen).float()
    a = void.void_from_block_mask(mask, tiles, device="cuda")
    b = torch.randint(-3, 4, (7 * 32, 200), generator=gen).float().cuda()
    gc = torch.randint(-3, 4, (9 * 32, 200), generator=gen).float().cuda()
    ref_v, ref_b = vo.spmm_backward(_np(a.values), _np(a.block_rows).astype(np.int32), _np(a.block_cols).astype(np.int32),
                                    a.shape, _np(b), _np(gc))
    for dt in (torch.float32, torch.float16, torch.bfloat16):
        got = void.spmm_tile_grad(a, gc.to(dt), b.to(dt), out_dtype=torch.float32)
        assert np.array_equal(_np(got), ref_v), dt
    a_t = void.VOIDTensor(a.values.permute(0, 2, 1).contiguous(), a.block_cols, a.block_rows, a.morton_codes,
                          (a.shape[1], a.shape[0]), (32, 32), 0, a.n_blocks, 0.0)
    assert np.array_equal(_np(void.void_spmm(a_t, gc)), ref_b)
    void.check_device_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_backward_vs_torch_dense_autograd(dtype):
    mask = workloads.uniform_mask(8, 8, 0.6, seed=5)
    w = workloads.block_sparse(mask, 96, seed=6)
    a = w.a.to_dtype(dtype)
    layer = void.VOIDSpMM(a, requires_grad=True)
    x = w.b.to(dtype).clone().requires_grad_(True)
    y = layer(x)
    gy = torch.randn(256, 96, device="cuda", generator=torch.Generator(device="cuda").manual_seed(2)).to(dtype)
    y.backward(gy)
    dense = a.to_dense().float().clone().requires_grad_(True)
    x_ref = w.b.to(dtype).float().clone().requires_grad_(True)
    (dense @ x_ref).backward(gy.float())
    tol = 1e-2 if dtype != torch.float32 else 2e-3
    assert rel_err(_np(y), _np(dense @ x_ref)) < tol
    assert rel_err(_np(x.grad), _np(x_ref.grad)) < tol
    got = _np(layer.values.grad)
    br, bc = _np(a.block_rows).astype(int), _np(a.block_cols).astype(int)
    full = _np(dense.grad)
    ref = np.stack([full[r * 32:(r + 1) * 32, c * 32:(c + 1) * 32] for r, c in zip(br, bc)])
    assert got.dtype == np.float32 and layer.values.grad.dtype == dtype and rel_err(got, ref) < tol


def test_gradients_at_benchmark_size(capsys):
    # 4096 x 4096 at 90 % block sparsity, N = 512: a sample of tile gradients and dB against dense products,
    # and the two kernels' device times (shown with pytest -s)
    w = workloads.headline(0.9, seed=0)
    gc = torch.randn(4096, 512, device="cuda", generator=torch.Generator(device="cuda").manual_seed(1))
    a_t = void.VOIDTensor(w.a.values.permute(0, 2, 1).contiguous(), w.a.block_cols, w.a.block_rows, w.a.morton_codes,
                          (4096, 4096), (32, 32), 0, w.a.n_blocks, 0.0)
    grad_tiles = void.spmm_tile_grad(w.a, gc, w.b)
    grad_b = void.void_spmm(a_t, gc)
    void.check_device_status()
    br, bc = _np(w.a.block_rows).astype(int), _np(w.a.block_cols).astype(int)
    for i in np.random.default_rng(0).choice(w.a.n_blocks, 24, replace=False):
        ref = gc[br[i] * 32:(br[i] + 1) * 32].double() @ w.b[bc[i] * 32:(bc[i] + 1) * 32].double().T
        assert rel_err(_np(grad_tiles[i]), _np(ref)) < 2e-3
    ref_b = w.a.to_dense().double().T[:, :1024] @ gc[:1024].double()
    full_b = w.a.to_dense().T @ gc
    assert rel_err(_np(grad_b), _np(full_b)) < 2e-3 and ref_b.shape == (4096, 512)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    for _ in range(3):
        void.spmm_tile_grad(w.a, gc, w.b)
        void.void_spmm(a_t, gc, grad_b)
    ev[0].record()
    for _ in range(20):
        void.spmm_tile_grad(w.a, gc, w.b)
    ev[1].record()
    for _ in range(20):
        void.void_spmm(a_t, gc, grad_b)
    ev[2].record()
    torch.cuda.synchronize()
    flops = 2.0 * w.a.n_blocks * 1024 * 512
    with capsys.disabled():
        print("\n[backward, 4096^2 90%% N=512 fp32] dA tiles %.1f us (%.1f TFLOP/s)  dB %.1f us (%.1f TFLOP/s)  "
              "(host-launched, L2-warm)" % (ev[0].elapsed_time(ev[1]) * 50, flops / (ev[0].elapsed_time(ev[1]) * 50e-6) / 1e12,
                                            ev[1].elapsed_time(ev[2]) * 50, flops / (ev[1].elapsed_time(ev[2]) * 50e-6) / 1e12))


def test_sparse_linear_gradients_vs_torch_linear():
    mask = workloads.uniform_mask(5, 7, 0.5, seed=4)
    w = workloads.block_sparse(mask, 8, seed=4)
    lin = void.SparseLinear(224, 160, w.a, bias=True)
    gen = torch.Generator(device="cuda").manual_seed(3)
    with torch.no_grad():
        lin.bias.copy_(torch.randn(160, device="cuda", generator=gen))
    x = torch.randn(3, 50, 224, device="cuda", generator=gen, requires_grad=True)
    gy = torch.randn(3, 50, 160, device="cuda", generator=gen)
    y = lin(x)
    y.backward(gy)
    dense = w.a.to_dense().clone().requires_grad_(True)
    x_ref = x.detach().clone().requires_grad_(True)
    b_ref = lin.bias.detach().clone().requires_grad_(True)
    torch.nn.functional.linear(x_ref, dense, b_ref).backward(gy)
    assert y.shape == (3, 50, 160) and y.is_contiguous()
    assert rel_err(_np(y), _np(torch.nn.functional.linear(x_ref, dense, b_ref))) < 2e-3
    assert rel_err(_np(x.grad), _np(x_ref.grad)) < 2e-3
    assert rel_err(_np(lin.bias.grad), _np(b_ref.grad)) < 1e-5
    br, bc = _np(w.a.block_rows).astype(int), _np(w.a.block_cols).astype(int)
    full = _np(dense.grad)
    ref = np.stack([full[r * 32:(r + 1) * 32, c * 32:(c + 1) * 32] for r, c in zip(br, bc)])
    assert rel_err(_np(lin.sparse_weight.values.grad), ref) < 2e-3
    void.check_device_status()


def test_sparse_linear_trains():
    # a few SGD steps on a regression target reduce the loss: gradients flow to the tiles and the bias
    mask = workloads.uniform_mask(4, 6, 0.5, seed=9)
    w = workloads.block_sparse(mask, 8, seed=9)
    lin = void.SparseLinear(192, 128, w.a, bias=True)
    assert [n for n, _ in lin.named_parameters()] == ["bias", "sparse_weight.values"]
    gen = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(4, 16, 192, device="cuda", generator=gen)
    target = torch.randn(4, 16, 128, device="cuda", generator=gen)
    opt = torch.optim.SGD(lin.parameters(), lr=1e-3)
    losses = []
    for _ in range(5):
        opt.zero_grad()
        y = lin(x)
        assert y.shape == (4, 16, 128)
        loss = torch.nn.functional.mse_loss(y, target)
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    assert losses[-1] < losses[0] and lin.bias.grad is not None and lin.sparse_weight.values.grad is not None
    y1 = void.VOIDSpMM(w.a, requires_grad=False)(w.b[:, 0])          # vector input, no parameters
    assert y1.shape == (128,) and rel_err(_np(y1), _np(w.a.to_dense() @ w.b[:, 0])) < 2e-3
    void.check_device_status()
