"""Numerics of every sm_100a kernel against a plain PyTorch fp32 restatement of the same op."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def _max_err(a, b):
    return (a.float() - b.float()).abs().max().item()


def _tile_errors(out, ref, tile=32):
    """Largest relative error of any `tile` x `tile` block: a missing or misplaced store box shows up here even when it
    vanishes in the norm of the whole matrix."""
    diff = (out.float() - ref.float())
    rows, cols = diff.shape
    pr, pc = (-rows) % tile, (-cols) % tile
    pad = lambda t: torch.nn.functional.pad(t, (0, pc, 0, pr))  # noqa: E731
    d = pad(diff).reshape((rows + pr) // tile, tile, (cols + pc) // tile, tile).pow(2).sum((1, 3)).sqrt()
    r = pad(ref.float()).reshape((rows + pr) // tile, tile, (cols + pc) // tile, tile).pow(2).sum((1, 3)).sqrt()
    return (d / (r + 1e-3 * r.max() + 1e-12)).max().item()


class _Guarded:
    """An output matrix inside a larger buffer whose surrounding rows and columns hold a sentinel: any store outside the
    matrix (a TMA box that is not clipped, a wrong leading dimension) changes a sentinel.  Stands in for a memory checker."""

    def __init__(self, rows, cols, dtype, margin=8, fill=None, sentinel=-7777.0):
        self.margin, self.sentinel = margin, sentinel
        align = 8 if dtype == torch.bfloat16 else 4
        ld = (cols + 2 * margin + align - 1) // align * align
        self.buffer = torch.full((rows + 2 * margin, ld), sentinel, device="cuda", dtype=dtype)
        self.view = self.buffer[margin : margin + rows, margin : margin + cols]
        if fill is not None:
            self.view.copy_(fill)
        self._inside = torch.zeros_like(self.buffer, dtype=torch.bool)
        self._inside[margin : margin + rows, margin : margin + cols] = True

    def check(self):
        outside = self.buffer[~self._inside]
        assert torch.all(outside == self.sentinel), f"{int((outside != self.sentinel).sum())} elements outside the output were overwritten"


@pytest.mark.parametrize("m,n,k", [(512, 768, 256), (1000, 520, 200), (130, 4104, 72), (384, 768, 320), (256, 264, 128)])
@pytest.mark.parametrize("block_n", [0, 128, 256, 512])
@pytest.mark.parametrize("epilogue", [0, 1, 2, 3])
def test_gemm_stays_inside_its_output_and_every_tile_is_right(m, n, k, block_n, epilogue):
    """All four epilogues (store / accumulate, bf16 / fp32) of every kernel, written into a guarded sub-matrix whose margin
    makes the TMA store boxes of edge tiles reach past the matrix: nothing outside may change, and every 32 x 32 block of
    the result must be right on its own (not only the matrix norm)."""
    from fast_llm_b200.ops.gemm import gemm_raw

    torch.manual_seed(m + n + k + epilogue)
    x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(n, k, device="cuda", dtype=torch.bfloat16)
    dtype = torch.float32 if epilogue in (1, 2) else torch.bfloat16
    base = torch.randn(m, n, device="cuda", dtype=dtype) if epilogue >= 2 else None
    guarded = _Guarded(m, n, dtype, fill=base)
    gemm_raw(x, w, guarded.view, m, n, k, False, False, epilogue, block_n=block_n)
    torch.cuda.synchronize()
    guarded.check()
    ref = x.float() @ w.float().t() + (base.float() if base is not None else 0)
    assert _rel_err(guarded.view, ref) < 1e-2
    assert _tile_errors(guarded.view, ref) < (4e-2 if dtype == torch.bfloat16 else 1e-2)
    assert _max_err(guarded.view, ref) < 0.02 * ref.abs().max().item() + 0.25


@pytest.fixture(scope="module", autouse=True)
def _lib_loaded():
    from fast_llm_b200.ops import _lib

    assert _lib.get_lib().flb_abi_version() == 1
    yield
    from fast_llm_b200.ops.gemm import check_device_errors

    check_device_errors()


GEMM_SHAPES = [(512, 768, 256), (1000, 520, 200), (128, 256, 64), (256, 512, 128), (384, 768, 320), (1024, 1024, 1024), (200, 328, 136), (8, 4096, 512),
               (4096, 1024, 4096), (130, 4104, 72)]


@pytest.mark.parametrize("m,n,k", GEMM_SHAPES)
@pytest.mark.parametrize("block_n", [0, 128, 256, 512])
def test_gemm_nt(m, n, k, block_n):
    from fast_llm_b200.ops.gemm import gemm_raw

    torch.manual_seed(0)
    x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(n, k, device="cuda", dtype=torch.bfloat16)
    out = torch.full((m, n), float("nan"), device="cuda", dtype=torch.bfloat16)
    gemm_raw(x, w, out, m, n, k, False, False, 0, block_n=block_n)
    ref = x.float() @ w.float().t()
    assert _rel_err(out, ref) < 1e-2
    assert torch.isfinite(out).all()


@pytest.mark.parametrize("m,n,k", GEMM_SHAPES)
def test_gemm_nn(m, n, k):
    from fast_llm_b200.ops.gemm import matmul_nn

    torch.manual_seed(1)
    dy = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(k, n, device="cuda", dtype=torch.bfloat16)
    out = matmul_nn(dy, w)
    ref = dy.float() @ w.float()
    assert _rel_err(out, ref) < 1e-2


@pytest.mark.parametrize("m,n,k", GEMM_SHAPES)
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gemm_tn_accumulate(m, n, k, out_dtype):
    from fast_llm_b200.ops.gemm import matmul_tn

    torch.manual_seed(2)
    dy = torch.randn(k, m, device="cuda", dtype=torch.bfloat16)
    x = torch.randn(k, n, device="cuda", dtype=torch.bfloat16)
    base = torch.randn(m, n, device="cuda", dtype=out_dtype)
    out = base.clone()
    matmul_tn(dy, x, out=out, accumulate=True)
    ref = base.float() + dy.float().t() @ x.float()
    assert _rel_err(out, ref) < (1e-2 if out_dtype == torch.bfloat16 else 2e-3)
    out2 = torch.empty(m, n, device="cuda", dtype=out_dtype)
    matmul_tn(dy, x, out=out2, accumulate=False)
    assert _rel_err(out2, dy.float().t() @ x.float()) < 1e-2


def test_gemm_mixed_majors_and_strided_views():
    from fast_llm_b200.ops.gemm import gemm_raw, matmul_nt

    torch.manual_seed(3)
    m, n, k = 256, 384, 192
    a_t = torch.randn(k, m, device="cuda", dtype=torch.bfloat16)  # A MN-major
    b = torch.randn(n, k, device="cuda", dtype=torch.bfloat16)  # B K-major
    out = torch.empty(m, n, device="cuda", dtype=torch.float32)
    gemm_raw(a_t, b, out, m, n, k, True, False, 1)
    assert _rel_err(out, a_t.float().t() @ b.float().t()) < 1e-2
    for block_n in (256, 512):
        gemm_raw(a_t, b, out.fill_(float("nan")), m, n, k, True, False, 1, block_n=block_n)
        assert _rel_err(out, a_t.float().t() @ b.float().t()) < 1e-2
    # operands that are column slices of wider buffers (leading dimension > logical width)
    big = torch.randn(m, 3 * k, device="cuda", dtype=torch.bfloat16)
    xs = big[:, k : 2 * k]
    outs = torch.empty(m, 2 * n, device="cuda", dtype=torch.bfloat16)
    matmul_nt(xs, b, out=outs[:, n:])
    assert _rel_err(outs[:, n:], xs.float() @ b.float().t()) < 1e-2


@pytest.mark.parametrize("rows,cols", [(64, 256), (300, 4096), (17, 8192), (5, 1000)])
@pytest.mark.parametrize("layer_norm", [False, True])
@pytest.mark.parametrize("zero_centered", [False, True])
def test_norm(rows, cols, layer_norm, zero_centered):
    from fast_llm_b200.ops.normalization import add_norm, norm, norm_reference

    torch.manual_seed(0)
    x = torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16)
    d = torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(cols, device="cuda") * 0.1 + (0 if zero_centered else 1)).bfloat16().requires_grad_()
    b = (torch.randn(cols, device="cuda") * 0.1).bfloat16().requires_grad_() if layer_norm else None
    xr, dr = x.clone().requires_grad_(), d.clone().requires_grad_()
    x.requires_grad_(), d.requires_grad_()
    res, y = add_norm(x, d, w, b, 1e-5, zero_centered, layer_norm)
    gy, gr = torch.randn_like(y), torch.randn_like(res)
    (y.float() * gy).sum().add((res.float() * gr).sum()).backward()
    wr = w.detach().float().requires_grad_()
    br = b.detach().float().requires_grad_() if b is not None else None
    res_r = (xr.float() + dr.float()).bfloat16().float()
    y_r = norm_reference(res_r, wr, br, 1e-5, zero_centered, layer_norm)
    ((y_r * gy).sum() + (res_r * gr).sum()).backward()
    assert _rel_err(y, y_r) < 1e-2
    assert _rel_err(res, res_r) < 1e-6
    assert _rel_err(x.grad, xr.grad) < 1.5e-2
    assert _rel_err(d.grad, dr.grad) < 1.5e-2
    assert _rel_err(w.grad, wr.grad) < 1.5e-2
    if b is not None:
        assert _rel_err(b.grad, br.grad) < 1.5e-2
    y2 = norm(x.detach(), w.detach(), None if b is None else b.detach(), 1e-5, zero_centered, layer_norm)
    assert _rel_err(y2, norm_reference(x.detach().float(), wr, br, 1e-5, zero_centered, layer_norm)) < 1e-2


def test_norm_grad_buffer_accumulation():
    from fast_llm_b200.ops.normalization import norm

    x = torch.randn(128, 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = torch.ones(512, device="cuda", dtype=torch.bfloat16)
    w.grad_buffer = torch.zeros(512, device="cuda", dtype=torch.float32)
    w.param_grad_is_zero = True
    for _ in range(2):
        norm(x, w).float().sum().backward()
    xf = x.detach().float()
    ref = 2 * (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5)).sum(0)
    assert _rel_err(w.grad_buffer, ref) < 1e-2
    assert w.param_grad_is_zero is False


@pytest.mark.parametrize("rot_dim", [128, 64])
def test_rope(rot_dim):
    from fast_llm_b200.ops.rotary import rope_, rope_reference

    torch.manual_seed(0)
    tokens, heads, kv, hd = 333, 8, 2, 128
    x = torch.randn(tokens, (heads + 2 * kv) * hd, device="cuda", dtype=torch.bfloat16)
    pos = torch.randint(0, 1000, (tokens,), device="cuda", dtype=torch.int32)
    ang = torch.arange(1000, device="cuda", dtype=torch.float64)[:, None] * (10000.0 ** (-torch.arange(0, rot_dim, 2, device="cuda", dtype=torch.float64) / rot_dim))[None]
    table = torch.cat([ang.cos(), ang.sin()], -1).float().contiguous()
    ref = rope_reference(x.float(), table, pos, heads + kv, hd, rot_dim)
    y = rope_(x.clone(), table, pos, heads + kv, hd, rot_dim)
    assert _rel_err(y, ref) < 5e-3
    assert torch.equal(y[:, (heads + kv) * hd :], x[:, (heads + kv) * hd :])
    back = rope_(y.clone(), table, pos, heads + kv, hd, rot_dim, conj=True)
    assert _rel_err(back, x) < 1e-2


@pytest.mark.parametrize("gated", [True, False])
@pytest.mark.parametrize("act", ["silu", "gelu", "relu", "squared_relu", "sigmoid", "identity", "gelu_erf"])
def test_mlp_activation(gated, act):
    from fast_llm_b200.ops.activation import ActivationType, mlp_activation, mlp_activation_reference

    torch.manual_seed(0)
    a = ActivationType(act)
    x = torch.randn(257, 1024, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    xr = x.detach().float().requires_grad_()
    y = mlp_activation(x, gated, a)
    yr = mlp_activation_reference(xr, gated, a)
    g = torch.randn_like(y)
    y.backward(g)
    yr.backward(g.float())
    assert _rel_err(y, yr) < 1e-2
    assert _rel_err(x.grad, xr.grad) < 1e-2


@pytest.mark.parametrize("b_mn", [False, True])
def test_gathered_and_scattered_gemm_modes_on_one_gpu(b_mn):
    """The two tensor-parallel modes of the CTA-pair GEMM with the peers' side played on the same GPU: arrival words already
    raised (the gathered GEMM starts at the "local" chunk and must still produce every row), and per-owner output maps that point
    at two local buffers (row blocks of chunk c must land in buffer c, nothing else touched)."""
    import ctypes

    from fast_llm_b200.ops import _lib
    from fast_llm_b200.ops.gemm import check_device_errors

    torch.manual_seed(0)
    lib = _lib.get_lib()
    rows, world, k, n = 512, 2, 384, 640
    a = torch.randn(rows * world, k, device="cuda", dtype=torch.bfloat16)
    w = torch.randn((k, n) if b_mn else (n, k), device="cuda", dtype=torch.bfloat16) / k**0.5
    reference = a.float() @ (w.float() if b_mn else w.float().t())
    # gathered: chunk 1 is "local", the arrival word of chunk 0 already holds the call number
    flags = torch.tensor([7, 0] + [0] * 14, device="cuda", dtype=torch.int32)
    out = torch.full((rows * world + 2, n), 3.0, device="cuda", dtype=torch.bfloat16)
    _lib.check(lib.flb_gemm_gathered_bf16(a.data_ptr(), w.data_ptr(), out[1:-1].data_ptr(), rows * world, n, k, k, w.stride(0), n, int(b_mn),
                                          flags.data_ptr(), 7, rows, 1, _lib.stream_ptr()), "flb_gemm_gathered_bf16")
    assert _rel_err(out[1:-1], reference) < 5e-3 and _max_err(out[1:-1], reference) < 0.1
    assert (out[0] == 3).all() and (out[-1] == 3).all()
    # scattered: chunk c -> buffer c
    buffers = torch.full((world, rows + 2, n), 5.0, device="cuda", dtype=torch.bfloat16)
    host = torch.empty(world * 128 + 64, dtype=torch.uint8)
    shift = (-host.data_ptr()) % 64
    aligned = host[shift : shift + world * 128]
    destinations = (ctypes.c_void_p * world)(*[buffers[c, 1:-1].data_ptr() for c in range(world)])
    _lib.check(lib.flb_gemm_scatter_maps(aligned.data_ptr(), destinations, world, rows, n, n), "flb_gemm_scatter_maps")
    device_buffer = torch.empty(world * 128 + 64, dtype=torch.uint8, device="cuda")
    device_shift = (-device_buffer.data_ptr()) % 64
    maps = device_buffer[device_shift : device_shift + world * 128]
    maps.copy_(aligned)
    torch.cuda.synchronize()
    _lib.check(lib.flb_gemm_scatter_bf16(a.data_ptr(), w.data_ptr(), maps.data_ptr(), rows * world, n, k, k, w.stride(0), int(b_mn), rows, 1,
                                         _lib.stream_ptr()), "flb_gemm_scatter_bf16")
    torch.cuda.synchronize()
    check_device_errors()
    for c in range(world):
        assert _rel_err(buffers[c, 1:-1], reference[c * rows : (c + 1) * rows]) < 5e-3, c
        assert (buffers[c, 0] == 5).all() and (buffers[c, -1] == 5).all()


def test_gemm_reuses_tensor_maps_for_repeated_operands():
    from fast_llm_b200.ops.gemm import matmul_nt, tensor_map_cache_stats

    x = torch.randn(512, 256, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(384, 256, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(512, 384, device="cuda", dtype=torch.bfloat16)
    matmul_nt(x, w, out=out)
    hits, misses = tensor_map_cache_stats()
    first = out.clone()
    matmul_nt(x, w, out=out)
    hits2, misses2 = tensor_map_cache_stats()
    assert misses2 == misses and hits2 >= hits + 3  # A, B and C maps all came from the table
    assert torch.equal(out, first)
    # another operand at the same address with another shape must not reuse a stale map
    matmul_nt(x[:256], w, out=out[:256])
    assert _rel_err(out[:256], x[:256].float() @ w.float().t()) < 5e-3


@pytest.mark.parametrize("m,f,k", [(512, 1024, 512), (1000, 328, 192), (4096, 3584, 1024), (257, 136, 64)])
@pytest.mark.parametrize("act", ["silu", "gelu"])
def test_gated_gemm_epilogue_matches_gemm_then_activation(m, f, k, act):
    """Layer-1 GEMM with the gated activation in its epilogue: `h` against an fp32 matmul, the activation output against
    the fp32 activation of the stored (bf16) `h`, and the whole MLP node (which takes this path) against its fp32 restatement."""
    from fast_llm_b200.ops.activation import ActivationType, mlp_activation_reference
    from fast_llm_b200.ops.gemm import gated_ok, matmul_nt_gated

    torch.manual_seed(0)
    a_type = ActivationType(act)
    x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    w1 = torch.randn(2 * f, k, device="cuda", dtype=torch.bfloat16) / k**0.5
    assert gated_ok(x, w1)
    h, a = matmul_nt_gated(x, w1, a_type.code)
    h_ref = x.float() @ w1.float().t()
    assert _rel_err(h, h_ref) < 5e-3
    a_ref = mlp_activation_reference(h.float(), True, a_type)
    assert _rel_err(a, a_ref) < 5e-3
    assert _max_err(a, a_ref) <= 2e-2 * a_ref.abs().max().item()


def test_mlp_node_with_fused_gated_epilogue_matches_fp32():
    from fast_llm_b200.ops.activation import ActivationType, mlp_activation_reference
    from fast_llm_b200.ops.mlp import MLPRecomputeLevel, mlp

    torch.manual_seed(0)
    m, k, f = 1024, 512, 768
    x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w1 = (torch.randn(2 * f, k, device="cuda", dtype=torch.bfloat16) / k**0.5).requires_grad_()
    w2 = (torch.randn(f, k, device="cuda", dtype=torch.bfloat16) / f**0.5).requires_grad_()
    for level in (MLPRecomputeLevel.none, MLPRecomputeLevel.activation, MLPRecomputeLevel.full):
        for t in (x, w1, w2):
            t.grad = None
            if hasattr(t, "grad_buffer"):
                del t.grad_buffer
        y = mlp(x, w1, None, w2, None, gated=True, activation=ActivationType.silu, recompute_level=level)
        g = torch.randn_like(y)
        y.backward(g)
        xr, w1r, w2r = (t.detach().float().requires_grad_() for t in (x, w1, w2))
        yr = mlp_activation_reference(xr @ w1r.t(), True, ActivationType.silu) @ w2r
        yr.backward(g.float())
        assert _rel_err(y, yr) < 1e-2
        assert _rel_err(x.grad, xr.grad) < 2e-2
        assert _rel_err(w1.grad, w1r.grad) < 2e-2
        assert _rel_err(w2.grad, w2r.grad) < 2e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("vocab", [32000, 1003])
def test_cross_entropy(dtype, vocab):
    from fast_llm_b200.ops.cross_entropy import cross_entropy_forward_backward, cross_entropy_reference

    torch.manual_seed(0)
    rows = 97
    ld = (vocab + 7) // 8 * 8
    buf = (torch.randn(rows, ld, device="cuda") * 3).to(dtype)
    logits = buf[:, :vocab]
    labels = torch.randint(0, vocab, (rows,), device="cuda")
    labels[::7] = -100
    loss_r, z_r, grad_r = cross_entropy_reference(logits.float(), labels, 0.37, 1.5, 1e-3)
    loss, z, grad = cross_entropy_forward_backward(logits, labels, 0.37, 1.5, 1e-3, in_place=False)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    assert _rel_err(loss, loss_r) < 1e-4
    assert _rel_err(z, z_r) < 1e-4
    assert _rel_err(grad, grad_r) < tol
    # sharded: two halves merged by hand must equal the unsharded result
    gs = torch.tensor([0.37], device="cuda")
    loss2, _, grad2 = cross_entropy_forward_backward(buf.clone()[:, :vocab], labels, gs, 1.5, 1e-3, in_place=True)
    assert _rel_err(loss2, loss_r) < 1e-4
    assert _rel_err(grad2, grad_r) < tol


def test_adamw_and_norm_kernels():
    from fast_llm_b200.ops.optim import adamw, adamw_reference, clip_coeff, sumsq

    torch.manual_seed(0)
    n = 1_000_003
    w = torch.randn(n + 1, device="cuda")[:n]
    n = (n // 4) * 4 + 3
    w = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda")
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    lp = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    wr, mr, vr = w.clone(), m.clone(), v.clone()
    nsq = torch.zeros(1, device="cuda")
    sumsq(g, nsq)
    assert abs(nsq.item() - g.double().pow(2).sum().item()) / nsq.item() < 1e-5
    coeff = torch.empty(1, device="cuda")
    norm = torch.empty(1, device="cuda")
    clip_coeff(nsq, 1.0, 0.5, coeff, norm)
    expect_norm = g.double().norm().item() * 0.5
    assert abs(norm.item() - expect_norm) / expect_norm < 1e-5
    expect_coeff = 0.5 * min(1.0, 1.0 / (expect_norm + 1e-6))
    assert abs(coeff.item() - expect_coeff) / expect_coeff < 1e-5
    for step in (1, 2, 3):
        adamw(w, g, m, v, lp, 1e-2, 0.9, 0.95, 1e-8, 0.1, step, 1.0, coeff)
        adamw_reference(wr, g, mr, vr, None, 1e-2, 0.9, 0.95, 1e-8, 0.1, step, expect_coeff)
    assert _rel_err(w, wr) < 1e-5
    assert _rel_err(m, mr) < 1e-5
    assert _rel_err(v, vr) < 1e-5
    assert torch.equal(lp, w.bfloat16())


def test_embedding_and_pointwise():
    from fast_llm_b200.ops.pointwise import axpby_, bias_residual, embedding, fill_

    torch.manual_seed(0)
    w = torch.randn(1000, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    ids = torch.randint(0, 1200, (4, 77), device="cuda")
    out = embedding(ids, w, 100, 1100, 2.0)
    mask = (ids >= 100) & (ids < 1100)
    ref = torch.nn.functional.embedding((ids - 100).clamp(0, 999), w.detach().float()) * mask[..., None] * 2.0
    assert _rel_err(out, ref) < 1e-2
    g = torch.randn_like(out)
    out.backward(g)
    wr = w.detach().float().requires_grad_()
    (torch.nn.functional.embedding((ids - 100).clamp(0, 999), wr) * mask[..., None] * 2.0 * g.float()).sum().backward()
    assert _rel_err(w.grad, wr.grad) < 1e-2
    a = torch.randn(100003, device="cuda")
    b = torch.randn(100003, device="cuda", dtype=torch.bfloat16)
    o = torch.empty(100003, device="cuda", dtype=torch.bfloat16)
    axpby_(o, a, b, 0.5, 2.0)
    assert _rel_err(o, a * 0.5 + b.float() * 2) < 1e-2
    fill_(o, 3.0)
    assert (o == 3).all()
    x = torch.randn(33, 512, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(512, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        r = bias_residual(x, bias, x, 0.5)
    assert _rel_err(r, (x.float() + bias.float()) * 0.5 + x.float()) < 1e-2


def _attention_case(doc_lengths, heads, kv_heads, causal, window, seed=0, variant=0):
    from fast_llm_b200.ops import _lib
    from fast_llm_b200.ops.attention import attention_forward_native, attention_reference

    torch.manual_seed(seed)
    d = 128
    total = sum(doc_lengths)
    qkv = torch.randn(total, (heads + 2 * kv_heads) * d, device="cuda", dtype=torch.bfloat16)
    cu = torch.tensor([0] + list(torch.tensor(doc_lengths).cumsum(0)), device="cuda", dtype=torch.int32)
    nq, nkv = heads * d, kv_heads * d
    old = _lib.get_lib().flb_attention_set_forward_variant(variant)
    try:
        out, lse = attention_forward_native(qkv, 0, qkv, nq, nq + nkv, cu, cu, max(doc_lengths), heads, kv_heads, d, causal, window, d**-0.5)
    finally:
        _lib.get_lib().flb_attention_set_forward_variant(old)
    q = qkv[:, :nq].reshape(total, heads, d)
    k = qkv[:, nq : nq + nkv].reshape(total, kv_heads, d)
    v = qkv[:, nq + nkv :].reshape(total, kv_heads, d)
    ref = attention_reference(q.float(), k.float(), v.float(), cu, cu, causal, window, d**-0.5)
    return out, lse, ref, (q, k, v, cu)


@pytest.mark.parametrize("doc_lengths,heads,kv_heads,causal,window", [
    ([128], 1, 1, True, None),
    ([256], 2, 1, True, None),
    ([1000], 4, 2, True, None),
    ([300, 77, 513, 1], 4, 2, True, None),
    ([1500], 4, 1, True, 256),
    ([700, 900], 8, 2, True, 100),
    ([640], 2, 2, False, None),
    ([2048], 8, 2, True, 1024),
])
@pytest.mark.parametrize("variant", [0, 1], ids=["p_in_tmem", "p_in_smem"])
def test_attention_forward_tcgen05(doc_lengths, heads, kv_heads, causal, window, variant):
    from fast_llm_b200.ops import _lib

    out, lse, ref, (q, k, v, cu) = _attention_case(doc_lengths, heads, kv_heads, causal, window, variant=variant)
    assert _lib.get_lib().flb_attention_error_word() == 0
    assert torch.isfinite(out).all()
    assert _rel_err(out, ref) < 1.5e-2
    assert _tile_errors(out.reshape(out.shape[0], -1), ref.reshape(ref.shape[0], -1)) < 6e-2
    # log-sum-exp against a direct computation for one head of the first document
    n = doc_lengths[0]
    s = (q[:n, 0].float() @ k[:n, 0].float().t()) * 128**-0.5
    i = torch.arange(n, device="cuda")
    mask = torch.ones(n, n, dtype=torch.bool, device="cuda")
    if causal:
        mask &= i[None, :] <= i[:, None]
    if window:
        mask &= i[None, :] > i[:, None] - window
    expected = torch.logsumexp(s.masked_fill(~mask, float("-inf")), -1)
    assert _rel_err(lse[0, :n], expected) < 2e-3


@pytest.mark.parametrize("doc_lengths,heads,kv_heads,causal,window", [
    ([128], 1, 1, True, None),
    ([256], 2, 1, True, None),
    ([1000], 4, 2, True, None),
    ([300, 77, 513, 1], 4, 2, True, None),
    ([1500], 4, 1, True, 256),
    ([700, 900], 8, 2, True, 100),
    ([640], 2, 2, False, None),
    ([2048], 8, 2, True, 1024),
])
def test_attention_backward_tcgen05(doc_lengths, heads, kv_heads, causal, window):
    """dq, dk, dv of the tcgen05 backward against autograd through the fp32 restatement."""
    from fast_llm_b200.ops import _lib
    from fast_llm_b200.ops.attention import attention_reference, packed_attention

    torch.manual_seed(3)
    d = 128
    total = sum(doc_lengths)
    nq, nkv = heads * d, kv_heads * d
    qkv = torch.randn(total, nq + 2 * nkv, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    cu = torch.tensor([0] + list(torch.tensor(doc_lengths).cumsum(0)), device="cuda", dtype=torch.int32)
    out = packed_attention(qkv, cu, max(doc_lengths), heads, kv_heads, d, causal=causal, window_size=window)
    g = torch.randn_like(out)
    out.backward(g)
    assert _lib.get_lib().flb_attention_bwd_error_word() == 0
    ref_in = qkv.detach().float().requires_grad_()
    ref = attention_reference(ref_in[:, :nq].reshape(total, heads, d), ref_in[:, nq : nq + nkv].reshape(total, kv_heads, d),
                              ref_in[:, nq + nkv :].reshape(total, kv_heads, d), cu, cu, causal, window, d**-0.5).reshape(total, nq)
    ref.backward(g.float())
    assert torch.isfinite(qkv.grad).all()
    for name, lo, hi in (("dq", 0, nq), ("dk", nq, nq + nkv), ("dv", nq + nkv, nq + 2 * nkv)):
        assert _rel_err(qkv.grad[:, lo:hi], ref_in.grad[:, lo:hi]) < 3e-2, name


def _prefix_case(q_lengths, k_lengths, heads, kv_heads, d, window, seed=5):
    torch.manual_seed(seed)
    tq, tk = sum(q_lengths), sum(k_lengths)
    q = torch.randn(tq, heads, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    kv = torch.randn(tk, 2 * kv_heads * d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    cu_q = torch.tensor([0] + list(torch.tensor(q_lengths).cumsum(0)), device="cuda", dtype=torch.int32)
    cu_k = torch.tensor([0] + list(torch.tensor(k_lengths).cumsum(0)), device="cuda", dtype=torch.int32)
    return q, kv, cu_q, cu_k


@pytest.mark.parametrize("q_lengths,k_lengths,heads,kv_heads,d,window", [
    ([128], [384], 2, 1, 128, None),          # a prefix of two key tiles
    ([200, 60], [456, 60], 4, 2, 128, None),  # one document with a prefix, one without
    ([300], [1000], 4, 2, 128, 256),          # prefix + sliding window
    ([257, 100], [300, 612], 2, 2, 128, None),
    ([384], [384], 4, 2, 64, None),           # head sizes below 128 are zero-padded
    ([300, 100], [500, 100], 4, 1, 96, 128),
])
def test_attention_with_key_prefix_and_padded_heads(q_lengths, k_lengths, heads, kv_heads, d, window):
    """General form: key segments longer than the query segments (bottom-right aligned causal mask), other head sizes;
    forward and all three gradients against the fp32 restatement."""
    from fast_llm_b200.ops import _lib
    from fast_llm_b200.ops.attention import attention, attention_reference

    q, kv, cu_q, cu_k = _prefix_case(q_lengths, k_lengths, heads, kv_heads, d, window)
    tk = kv.shape[0]
    k = kv[:, : kv_heads * d].reshape(tk, kv_heads, d)
    v = kv[:, kv_heads * d :].reshape(tk, kv_heads, d)
    before = _lib.launch_count
    out = attention(q, k, v, cu_q, cu_k, max(q_lengths), max(k_lengths), causal=True, window_size=window)
    g = torch.randn_like(out)
    out.backward(g)
    assert _lib.launch_count - before == 4, "forward + delta / backward / dq-convert kernels of this library"
    assert _lib.get_lib().flb_attention_error_word() == 0 and _lib.get_lib().flb_attention_bwd_error_word() == 0
    q32, kv32 = q.detach().float().requires_grad_(), kv.detach().float().requires_grad_()
    ref = attention_reference(q32, kv32[:, : kv_heads * d].reshape(tk, kv_heads, d), kv32[:, kv_heads * d :].reshape(tk, kv_heads, d), cu_q, cu_k,
                              True, window, d**-0.5)
    ref.backward(g.float())
    assert _rel_err(out, ref) < 1.5e-2
    assert _max_err(out, ref) < 0.05 * ref.abs().max().item()
    assert _rel_err(q.grad, q32.grad) < 3e-2
    assert _rel_err(kv.grad, kv32.grad) < 3e-2


def test_attention_key_rows_outside_every_document_get_zero_gradient():
    """Sequence-data parallelism hands every rank the whole key / value tensor; rows past the last `cu_k` belong to later
    tokens of other ranks and must come back with an exactly zero gradient."""
    from fast_llm_b200.ops.attention import attention

    heads, kv_heads, d = 2, 1, 128
    q, kv, cu_q, cu_k = _prefix_case([256], [512], heads, kv_heads, d, None)
    kv_long = torch.cat([kv.detach(), torch.randn(300, 2 * kv_heads * d, device="cuda", dtype=torch.bfloat16)]).requires_grad_()
    tk = kv_long.shape[0]
    out = attention(q, kv_long[:, : kv_heads * d].reshape(tk, kv_heads, d), kv_long[:, kv_heads * d :].reshape(tk, kv_heads, d), cu_q, cu_k, 256, 512)
    out.sum().backward()
    assert torch.all(kv_long.grad[512:] == 0)
    assert kv_long.grad[:512].abs().sum() > 0


def test_attention_dropout_fallback_keeps_the_expectation():
    """Dropout goes through the per-document PyTorch path: with p = 0 it equals the kernels, with p > 0 the mean over many
    masks approaches the undropped output."""
    from fast_llm_b200.ops.attention import attention

    heads, kv_heads, d = 2, 1, 128
    q, kv, cu_q, cu_k = _prefix_case([128], [128], heads, kv_heads, d, None)
    k = kv[:, : kv_heads * d].reshape(128, kv_heads, d)
    v = kv[:, kv_heads * d :].reshape(128, kv_heads, d)
    with torch.no_grad():
        exact = attention(q, k, v, cu_q, cu_k, 128, 128).float()
        mean = torch.zeros_like(exact)
        runs = 200
        for _ in range(runs):
            mean += attention(q, k, v, cu_q, cu_k, 128, 128, dropout_p=0.2).float() / runs
    assert _rel_err(mean, exact) < 0.15


@pytest.mark.parametrize("tokens,experts,k", [(300, 8, 2), (1000, 64, 8), (257, 4, 1), (8192, 8, 2)])
def test_moe_routing_kernels_match_the_restatement(tokens, experts, k):
    """Scores, chosen experts, load-balancing and z-loss values, and the logit gradient (score gradients plus both auxiliary
    losses) of the routing kernels against the PyTorch restatement."""
    from fast_llm_b200.ops.moe_routing import route_topk, route_topk_reference

    torch.manual_seed(tokens + experts)
    logits = torch.randn(tokens, experts, device="cuda") * 2
    upstream = torch.randn(tokens, k, device="cuda")
    results = []
    for fn in (route_topk, route_topk_reference):
        x = logits.clone().requires_grad_()
        scores, top, aux, z = fn(x, k, 0.3, 0.05)
        (scores * upstream).sum().backward()
        results.append((scores.detach(), top.long(), aux, z, x.grad))
    (s_a, t_a, aux_a, z_a, g_a), (s_b, t_b, aux_b, z_b, g_b) = results
    assert torch.equal(t_a, t_b)
    torch.testing.assert_close(s_a, s_b, rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(aux_a, aux_b, rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(z_a, z_b, rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(g_a, g_b, rtol=2e-3, atol=2e-6)


@pytest.mark.parametrize("tokens,experts,k", [(700, 4, 2), (513, 64, 8), (8192, 8, 2), (5, 3, 1)])
def test_moe_layout_kernel_matches_the_sort_based_layout(tokens, experts, k):
    from fast_llm_b200.ops.grouped_gemm import TILE_ROWS, expert_rows
    from fast_llm_b200.ops.moe_routing import expert_rows_native

    top, _ = _expert_layout_case(tokens, k, experts)
    rows_a, begin_a, upper_a = expert_rows_native(top.to(torch.int32), experts, TILE_ROWS)
    rows_b, begin_b, upper_b = expert_rows(top, experts)
    assert torch.equal(rows_a, rows_b) and torch.equal(begin_a, begin_b) and upper_a == upper_b


def _expert_layout_case(tokens, k, experts, seed=0):
    from fast_llm_b200.ops.grouped_gemm import expert_layout

    torch.manual_seed(seed)
    top = torch.stack([torch.randperm(experts, device="cuda")[:k] for _ in range(tokens)])
    if experts > 2:
        top[top == experts - 1] = 0  # leave the last expert without tokens
    return top, expert_layout(top, experts)


@pytest.mark.parametrize("b_mn", [False, True])
def test_grouped_gemm_rows(b_mn):
    from fast_llm_b200.ops.grouped_gemm import grouped_rows

    experts, n, k = 4, 384, 192
    top, (token_index, dest, row_begin, rows, order) = _expert_layout_case(700, 2, experts)
    a = torch.zeros(rows, k, device="cuda", dtype=torch.bfloat16)
    a[dest] = torch.randn(dest.numel(), k, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(experts * (k if b_mn else n), n if b_mn else k, device="cuda", dtype=torch.bfloat16)
    out = grouped_rows(a, b, row_begin, experts, n, k, b_mn)
    begins = row_begin.tolist()
    for e in range(experts):
        lo, hi = begins[e], begins[e + 1]
        if hi == lo:
            continue
        w = b[e * k : (e + 1) * k].float() if b_mn else b[e * n : (e + 1) * n].float().t()
        assert _rel_err(out[lo:hi], a[lo:hi].float() @ w) < 1e-2, e
    from fast_llm_b200.ops.gemm import check_device_errors

    check_device_errors()


@pytest.mark.parametrize("accumulate,dtype", [(False, torch.float32), (True, torch.float32), (False, torch.bfloat16)])
def test_grouped_gemm_wgrad(accumulate, dtype):
    from fast_llm_b200.ops.grouped_gemm import grouped_wgrad

    experts, m, n = 4, 256, 192
    top, (token_index, dest, row_begin, rows, order) = _expert_layout_case(900, 2, experts, seed=1)
    a = torch.zeros(rows, m, device="cuda", dtype=torch.bfloat16)
    b = torch.zeros(rows, n, device="cuda", dtype=torch.bfloat16)
    a[dest] = torch.randn(dest.numel(), m, device="cuda", dtype=torch.bfloat16)
    b[dest] = torch.randn(dest.numel(), n, device="cuda", dtype=torch.bfloat16)
    start = torch.randn(experts * m, n, device="cuda", dtype=dtype)
    out = start.clone()
    grouped_wgrad(a, b, out, row_begin, experts, accumulate)
    begins = row_begin.tolist()
    for e in range(experts):
        lo, hi = begins[e], begins[e + 1]
        expected = a[lo:hi].float().t() @ b[lo:hi].float()
        if accumulate:
            expected = expected + start[e * m : (e + 1) * m].float()
        got = out[e * m : (e + 1) * m].float()
        if hi == lo and not accumulate:
            assert (got == 0).all(), "an expert without rows must produce a zero gradient"
        else:
            assert _rel_err(got, expected) < 2e-2, e


def test_moe_grouped_matches_looped():
    """The MoE layer on the grouped tcgen05 GEMMs against the per-expert loop: outputs, input and weight gradients."""
    import fast_llm_b200.models.auto  # noqa: F401
    from fast_llm_b200.layers.moe import MoEMLPConfig
    from fast_llm_b200.parallel.topology import DistributedConfig
    from fast_llm_b200.tensor import TensorDim

    def build(implementation):
        config = MoEMLPConfig.from_dict({"type": "moe", "experts": 4, "experts_per_token": 2, "intermediate_size": 256, "gated": True,
                                         "activation": "silu", "add_linear_biases": False, "implementation": implementation})
        config.validate()
        distributed_config = DistributedConfig.from_dict({"compute_dtype": "bf16", "seed": 0, "world_size": 1, "rank": 0, "local_world_size": 1})
        distributed_config.validate()
        layer = config.get_layer(distributed_config, TensorDim("hidden", 128))
        layer.set_names("mlp.")
        return layer.materialize(device=torch.device("cuda"), dtype=torch.bfloat16)

    grouped, looped = build("dropless"), build("looped")
    for (_, a), (_, b) in zip(grouped.named_parameter_metas(), looped.named_parameter_metas()):
        b.tensor.data.copy_(a.tensor.data)
    torch.manual_seed(0)
    x = torch.randn(600, 128, device="cuda", dtype=torch.bfloat16)
    g = torch.randn(600, 128, device="cuda", dtype=torch.bfloat16)
    results = []
    for layer in (grouped, looped):
        xi = x.clone().requires_grad_()
        y = layer.forward(xi, {"training": True})
        y.backward(g)
        results.append((y.detach().float(), xi.grad.float(), {n: m.tensor.grad.float() for n, m in layer.named_parameter_metas() if m.tensor.grad is not None}))
    (y0, dx0, w0), (y1, dx1, w1) = results
    assert _rel_err(y0, y1) < 2e-2 and _rel_err(dx0, dx1) < 3e-2
    assert set(w0) == set(w1) and {"layer_1.weight", "layer_2.weight"} <= set(w0)
    for name in w0:
        assert _rel_err(w0[name], w1[name]) < 3e-2, name


@pytest.mark.parametrize("tokens,channels,width,act,with_docs", [(1000, 64, 4, "silu", True), (257, 136, 3, "identity", False), (33, 8, 8, "gelu", True)])
def test_causal_conv1d(tokens, channels, width, act, with_docs):
    from fast_llm_b200.ops.activation import ActivationType
    from fast_llm_b200.ops.ssm import causal_conv1d, causal_conv1d_reference

    torch.manual_seed(0)
    x = torch.randn(tokens, channels, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(channels, width, device="cuda") * 0.5).bfloat16().requires_grad_()
    b = torch.randn(channels, device="cuda").bfloat16().requires_grad_()
    doc = torch.sort(torch.randint(0, 5, (tokens,), device="cuda")).values.int() if with_docs else None
    g = torch.randn(tokens, channels, device="cuda", dtype=torch.bfloat16)
    out = causal_conv1d(x, w, b, doc, ActivationType(act))
    out.backward(g)
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, b))
    ref = causal_conv1d_reference(xr, wr, br, doc, ActivationType(act))
    ref.backward(g.float())
    assert _rel_err(out, ref) < 1e-2
    assert _rel_err(x.grad, xr.grad) < 2e-2
    assert _rel_err(w.grad, wr.grad) < 2e-2
    assert _rel_err(b.grad, br.grad) < 2e-2


@pytest.mark.parametrize("tokens,channels,state,groups_b,groups_c,gated,docs", [
    (200, 64, 16, 2, 4, True, [0, 70, 71, 200]), (130, 32, 8, 1, 4, False, None), (64, 128, 16, 8, 8, True, [0, 64]), (300, 32, 4, 1, 1, True, [0, 129, 300]), (97, 384, 16, 2, 24, True, [0, 50, 97]), (70, 256, 32, 4, 8, False, None)])
def test_selective_scan_kernel(tokens, channels, state, groups_b, groups_c, gated, docs):
    from fast_llm_b200.ops.ssm import _SelectiveScan, document_starts, selective_scan, selective_scan_reference

    torch.manual_seed(0)
    dev = "cuda"
    x = torch.randn(tokens, channels, device=dev).bfloat16().requires_grad_()
    dt = (torch.randn(tokens, channels, device=dev) - 1).bfloat16().requires_grad_()
    a = (-torch.rand(channels, state, device=dev) * 2 - 0.1).requires_grad_()
    b = torch.randn(tokens, groups_b, state, device=dev).bfloat16().requires_grad_()
    c = torch.randn(tokens, groups_c, state, device=dev).bfloat16().requires_grad_()
    skip = torch.randn(channels, device=dev).requires_grad_()
    z = torch.randn(tokens, channels, device=dev).bfloat16().requires_grad_() if gated else None
    bias = torch.randn(channels, device=dev).requires_grad_()
    cu = None if docs is None else torch.tensor(docs, device=dev, dtype=torch.int32)
    g = torch.randn(tokens, channels, device=dev).bfloat16()
    inputs = [x, dt, a, b, c, skip] + ([z] if gated else []) + [bias]
    out = selective_scan(x, dt, a, b, c, skip, z, bias, cu)
    assert out.grad_fn is not None and type(out.grad_fn).__name__.startswith("_SelectiveScan")
    out.backward(g)
    refs = [t.detach().float().requires_grad_() for t in inputs]
    rz = refs[6] if gated else None
    ref = selective_scan_reference(refs[0], refs[1], refs[2], refs[3], refs[4], refs[5], rz, refs[-1], cu)
    ref.backward(g.float())
    assert _rel_err(out, ref) < 1e-2
    for name, t, r in zip(["x", "dt", "a", "b", "c", "skip"] + (["z"] if gated else []) + ["bias"], inputs, refs):
        assert _rel_err(t.grad, r.grad) < 2e-2, name


@pytest.mark.parametrize("per_channel", [False, True])
def test_delta_rule_state_scan_kernel(per_channel):
    """Gated DeltaNet / KDA recurrence on the GPU path (batched chunk-local work + the state-scan kernel and its adjoint)
    against the token-by-token fp32 restatement, with documents."""
    from fast_llm_b200.ops.ssm import _DeltaStateScan, chunk_delta_rule, delta_rule_reference

    torch.manual_seed(0)
    tokens, heads, dim = 300, 4, 64
    dev = "cuda"
    q, k, v = (torch.randn(tokens, heads, dim, device=dev).bfloat16().requires_grad_() for _ in range(3))
    g = (-torch.rand((tokens, heads, dim) if per_channel else (tokens, heads), device=dev) * 0.2).requires_grad_()
    beta = torch.rand(tokens, heads, device=dev).requires_grad_()
    cu = torch.tensor([0, 70, 200, 300], device=dev, dtype=torch.int32)
    grad_out = torch.randn(tokens, heads, dim, device=dev).bfloat16()
    assert _DeltaStateScan.applies(torch.empty(1, heads, dim, dim, device=dev), torch.empty(1, heads, dim, dim, device=dev))
    out = chunk_delta_rule(q, k, v, g, beta, cu)
    grads = torch.autograd.grad(out, (q, k, v, g, beta), grad_out)
    reference_inputs = [t.detach().float().requires_grad_() for t in (q, k, v, g, beta)]
    reference = delta_rule_reference(*reference_inputs, cu)
    reference_grads = torch.autograd.grad(reference, reference_inputs, grad_out.float())
    assert _rel_err(out, reference) < 1e-2
    for name, a, b in zip("q k v g beta".split(), grads, reference_grads):
        assert _rel_err(a, b) < 1e-2, name
