"""Kernel micro-benchmarks: device time (CUDA events, L2 flushed between iterations) and fraction of the measured peaks.

Counterpart of the reference's `tools/benchmark/triton_kernels/` harness.  Usage:
    python -m fast_llm_b200.tools.bench_kernels [--json out.json] [gemm] [elementwise]
Peaks come from MEASURED_PEAKS.json at the repository root when present, else the stated fallbacks.
"""

import json
import pathlib
import sys

import torch


def _peaks():
    path = pathlib.Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def time_op(fn, iters=10, warmup=3):
    """Median device time of `fn` in ms.  All iterations are queued without a host synchronisation in between: each one writes a
    1 GiB buffer (an L2 flush that also keeps the GPU busy while the host queues the next launches), then records an event,
    runs `fn` and records another event - so the interval holds the kernels of `fn` and not the host's launch latency."""
    flush = torch.empty(1024 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    pairs = []
    for _ in range(iters):
        flush.zero_()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        end.record()
        pairs.append((start, end))
    torch.cuda.synchronize()
    times = sorted(start.elapsed_time(end) for start, end in pairs)
    return times[len(times) // 2]


def bench_gemm(results):
    from fast_llm_b200.ops.gemm import matmul_nn, matmul_nt, matmul_tn

    _, tflops_peak, kind = _peaks()
    t = 8192
    shapes = [("qkv", 4096, 6144), ("dense", 4096, 4096), ("mlp1", 4096, 28672), ("mlp2", 14336, 4096), ("head", 4096, 32000)]
    for name, k, n in shapes:
        x = torch.randn(t, k, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(n, k, device="cuda", dtype=torch.bfloat16)
        dy = torch.randn(t, n, device="cuda", dtype=torch.bfloat16)
        gw = torch.zeros(n, k, device="cuda", dtype=torch.float32)
        flops = 2.0 * t * k * n
        rows = {
            "fprop": (lambda: matmul_nt(x, w), lambda: torch.matmul(x, w.t())),
            "dgrad": (lambda: matmul_nn(dy, w), lambda: torch.matmul(dy, w)),
            "wgrad_acc_f32": (lambda: matmul_tn(dy, x, out=gw, accumulate=True), lambda: gw.addmm_(dy.t(), x) if False else torch.matmul(dy.t(), x)),
        }
        for kind_name, (ours, lib) in rows.items():
            ms = time_op(ours)
            ms_lib = time_op(lib)
            r = {"op": f"gemm_{name}_{kind_name}", "shape": [t, n, k], "ms": ms, "tflops": flops / ms / 1e9,
                 "frac_of_peak": flops / ms / 1e9 / tflops_peak, "peak_kind": kind, "cublas_ms": ms_lib,
                 "cublas_tflops": flops / ms_lib / 1e9}
            results.append(r)
            print(json.dumps(r), flush=True)
        del x, w, dy, gw


def bench_elementwise(results):
    from fast_llm_b200.ops.activation import ActivationType, act_bwd_native, act_fwd_native
    from fast_llm_b200.ops.cross_entropy import cross_entropy_forward_backward
    from fast_llm_b200.ops.normalization import _bwd_native, _fwd_native
    from fast_llm_b200.ops.optim import adamw
    from fast_llm_b200.ops.rotary import rope_

    gbs_peak, _, kind = _peaks()
    t, h, f = 8192, 4096, 14336

    def rec(name, nbytes, fn):
        ms = time_op(fn)
        r = {"op": name, "ms": ms, "gbs": nbytes / ms / 1e6, "frac_of_peak": nbytes / ms / 1e6 / gbs_peak, "peak_kind": kind}
        results.append(r)
        print(json.dumps(r), flush=True)

    x = torch.randn(t, h, device="cuda", dtype=torch.bfloat16)
    d = torch.randn(t, h, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(h, device="cuda", dtype=torch.bfloat16)
    rec("add_rmsnorm_fwd", 4 * t * h * 2, lambda: _fwd_native(x, d, w, None, 1e-5, False, False))
    _, y, rstd, _ = _fwd_native(x, d, w, None, 1e-5, False, False)
    rec("rmsnorm_bwd", 4 * t * h * 2, lambda: _bwd_native(y, x, w, None, rstd, None, d, False, False, True))
    gu = torch.randn(t, 2 * f, device="cuda", dtype=torch.bfloat16)
    go = torch.randn(t, f, device="cuda", dtype=torch.bfloat16)
    rec("swiglu_fwd", 3 * t * f * 2, lambda: act_fwd_native(gu, True, ActivationType.silu))
    rec("swiglu_bwd_recompute", 6 * t * f * 2, lambda: act_bwd_native(go, gu, True, ActivationType.silu, True))
    # layer-1 GEMM with the gated activation in its epilogue against the GEMM followed by the activation kernel
    from fast_llm_b200.ops.gemm import matmul_nt, matmul_nt_gated

    w1 = torch.randn(2 * f, h, device="cuda", dtype=torch.bfloat16) / h**0.5
    fused_ms = time_op(lambda: matmul_nt_gated(x, w1, ActivationType.silu.code))
    split_ms = time_op(lambda: act_fwd_native(matmul_nt(x, w1), True, ActivationType.silu))
    r = {"op": "mlp1_gated_fprop", "shape": [t, 2 * f, h], "fused_ms": fused_ms, "gemm_then_activation_ms": split_ms,
         "tflops_fused": 2.0 * t * 2 * f * h / fused_ms / 1e9}
    results.append(r)
    print(json.dumps(r), flush=True)
    qkv = torch.randn(t, 6144, device="cuda", dtype=torch.bfloat16)
    ang = torch.arange(t, device="cuda", dtype=torch.float64)[:, None] * (10000.0 ** (-torch.arange(0, 128, 2, device="cuda", dtype=torch.float64) / 128))[None]
    table = torch.cat([ang.cos(), ang.sin()], -1).float().contiguous()
    rec("rope_qk", 2 * t * 5120 * 2, lambda: rope_(qkv, table, None, 40, 128, 128))
    logits = torch.randn(t, 32000, device="cuda", dtype=torch.bfloat16)
    labels = torch.randint(0, 32000, (t,), device="cuda")
    rec("cross_entropy_fwd_bwd", 3 * t * 32000 * 2, lambda: cross_entropy_forward_backward(logits, labels, 1.0, in_place=False))
    n = 256 * 1024 * 1024
    pw, pg, pm, pv = (torch.zeros(n, device="cuda") for _ in range(4))
    lp = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    rec("adamw", n * 30, lambda: adamw(pw, pg, pm, pv, lp, 1e-3, 0.9, 0.95, 1e-8, 0.1, 1))


def bench_gemm_tiles(results):
    """Same GEMM with 128- and 256-wide tiles: separates tensor-pipe limits from operand-feed (L2 -> SMEM) limits."""
    from fast_llm_b200.ops.gemm import gemm_raw

    _, tflops_peak, kind = _peaks()
    t, k, n = 8192, 4096, 6144
    x = torch.randn(t, k, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(n, k, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(t, n, device="cuda", dtype=torch.bfloat16)
    for block_n in (128, 256, 512):
        for max_ctas in (0, 74):
            ms = time_op(lambda: gemm_raw(x, w, out, t, n, k, False, False, 0, block_n=block_n, max_ctas=max_ctas))
            r = {"op": f"gemm_fprop_bn{block_n}_ctas{max_ctas or 148}", "shape": [t, n, k], "ms": ms, "tflops": 2.0 * t * n * k / ms / 1e9,
                 "frac_of_peak": 2.0 * t * n * k / ms / 1e9 / tflops_peak, "peak_kind": kind, "cublas_ms": float("nan"), "cublas_tflops": float("nan")}
            results.append(r)
            print(json.dumps(r), flush=True)


def bench_attention(results):
    """Attention at the Mistral-7B shape (8192 tokens, 32/8 heads, window 4096): both forward kernels and the backward."""
    from fast_llm_b200.ops import _lib
    from fast_llm_b200.ops.attention import attention_backward_native, attention_forward_native

    _, tflops_peak, kind = _peaks()
    t, heads, kv, d, window = 8192, 32, 8, 128, 4096
    qkv = torch.randn(t, (heads + 2 * kv) * d, device="cuda", dtype=torch.bfloat16)
    cu = torch.tensor([0, t], device="cuda", dtype=torch.int32)
    nq, nkv = heads * d, kv * d
    keys = (window * (window + 1) / 2 + (t - window) * window) / t  # average keys per query
    flops = 4.0 * t * keys * heads * d
    ours = lambda: attention_forward_native(qkv, 0, qkv, nq, nq + nkv, cu, cu, t, heads, kv, d, True, window, d**-0.5)
    lib = _lib.get_lib()
    for variant, name in ((0, "p_in_tmem"), (1, "p_in_smem")):
        old = lib.flb_attention_set_forward_variant(variant)
        ms = time_op(ours)
        lib.flb_attention_set_forward_variant(old)
        r = {"op": f"attention_fwd_mistral_{name}", "ms": ms, "tflops": flops / ms / 1e9, "frac_of_peak": flops / ms / 1e9 / tflops_peak,
             "peak_kind": kind, "cublas_ms": float("nan"), "cublas_tflops": float("nan")}
        results.append(r)
        print(json.dumps(r), flush=True)
    # backward: 2.5x the forward FLOPs (five tile products against two)
    out, lse = ours()
    dout = torch.randn(t, nq, device="cuda", dtype=torch.bfloat16)
    dqkv = torch.empty_like(qkv)
    ours_b = lambda: attention_backward_native(qkv, 0, qkv, nq, nq + nkv, out, dout, lse, cu, cu, t, heads, kv, d, dqkv, dqkv, True, window, d**-0.5)
    ms = time_op(ours_b)
    r = {"op": "attention_bwd_mistral", "ms": ms, "tflops": 2.5 * flops / ms / 1e9, "frac_of_peak": 2.5 * flops / ms / 1e9 / tflops_peak,
         "peak_kind": kind, "cublas_ms": float("nan"), "cublas_tflops": float("nan")}
    results.append(r)
    print(json.dumps(r), flush=True)


def bench_moe(results):
    """Mixtral-8x7B MLP layer (hidden 4096, ffn 14336, 8 experts, top-2) at 8192 tokens, forward + backward: grouped
    tcgen05 GEMMs against the per-expert loop."""
    import fast_llm_b200.models.auto  # noqa: F401
    from fast_llm_b200.layers.moe import MoEMLPConfig
    from fast_llm_b200.parallel.topology import DistributedConfig
    from fast_llm_b200.tensor import TensorDim

    _, tflops_peak, kind = _peaks()
    tokens, hidden, ffn, experts, top_k = 8192, 4096, 14336, 8, 2

    def build(implementation):
        config = MoEMLPConfig.from_dict({"type": "moe", "experts": experts, "experts_per_token": top_k, "intermediate_size": ffn, "gated": True,
                                         "activation": "silu", "add_linear_biases": False, "implementation": implementation})
        config.validate()
        dc = DistributedConfig.from_dict({"compute_dtype": "bf16", "seed": 0, "world_size": 1, "rank": 0, "local_world_size": 1})
        dc.validate()
        layer = config.get_layer(dc, TensorDim("hidden", hidden))
        layer.set_names("mlp.")
        return layer.materialize(device=torch.device("cuda"), dtype=torch.bfloat16)

    x = torch.randn(tokens, hidden, device="cuda", dtype=torch.bfloat16)
    g = torch.randn(tokens, hidden, device="cuda", dtype=torch.bfloat16)
    flops = 3 * 2.0 * tokens * top_k * hidden * ffn * 3  # three products of [rows, hidden] x [hidden, ffn] per direction, fwd + 2x bwd
    timings = {}
    for implementation in ("dropless", "looped"):
        layer = build(implementation)

        def step():
            xi = x.detach().requires_grad_()
            layer.forward(xi, {"training": True}).backward(g)
            for _, meta in layer.named_parameter_metas():
                meta.tensor.grad = None

        timings[implementation] = time_op(step)
        del layer
        torch.cuda.empty_cache()
    ms, ms_loop = timings["dropless"], timings["looped"]
    r = {"op": "moe_mixtral_layer_fwd_bwd", "ms": ms, "tflops": flops / ms / 1e9, "frac_of_peak": flops / ms / 1e9 / tflops_peak, "peak_kind": kind,
         "cublas_ms": ms_loop, "cublas_tflops": flops / ms_loop / 1e9, "note": "second pair = per-expert loop on the same tcgen05 GEMM (host sync per layer)"}
    results.append(r)
    print(json.dumps(r), flush=True)


def bench_ssm(results):
    """Mamba mixer inner ops at 8192 tokens, d_inner 4096, state 16: causal conv1d and selective scan, forward and backward.
    The scan is bounded by exp throughput (tokens x channels x state exponentials per pass), not by HBM: both are reported."""
    from fast_llm_b200.ops.activation import ActivationType
    from fast_llm_b200.ops.ssm import causal_conv1d, selective_scan

    hbm, _, kind = _peaks()
    tokens, channels, state, groups = 8192, 4096, 16, 32
    dev = "cuda"
    x = torch.randn(tokens, channels, device=dev).bfloat16().requires_grad_()
    w = torch.randn(channels, 4, device=dev).bfloat16().requires_grad_()
    bias = torch.randn(channels, device=dev).bfloat16().requires_grad_()
    g = torch.randn(tokens, channels, device=dev).bfloat16()
    silu = ActivationType("silu")
    out = [None]

    def conv_fwd():
        out[0] = causal_conv1d(x, w, bias, None, silu)

    ms = time_op(conv_fwd)
    nbytes = 2 * tokens * channels * 2
    r = {"op": "causal_conv1d_fwd", "ms": ms, "gbs": nbytes / ms / 1e6, "frac_of_peak": nbytes / ms / 1e6 / hbm, "peak_kind": kind}
    results.append(r)
    print(json.dumps(r), flush=True)
    ms = time_op(lambda: torch.autograd.grad(out[0], (x, w, bias), g, retain_graph=True))
    nbytes = 6 * tokens * channels * 2  # x, dout -> dpre; dpre -> dx; x, dpre -> dw
    r = {"op": "causal_conv1d_bwd", "ms": ms, "gbs": nbytes / ms / 1e6, "frac_of_peak": nbytes / ms / 1e6 / hbm, "peak_kind": kind}
    results.append(r)
    print(json.dumps(r), flush=True)

    dt = (torch.randn(tokens, channels, device=dev) - 1).bfloat16().requires_grad_()
    z = torch.randn(tokens, channels, device=dev).bfloat16().requires_grad_()
    a = (-torch.rand(channels, state, device=dev) - 0.1).requires_grad_()
    b = torch.randn(tokens, groups, state, device=dev).bfloat16().requires_grad_()
    c = torch.randn(tokens, channels // state, state, device=dev).bfloat16().requires_grad_()
    skip = torch.randn(channels, device=dev).requires_grad_()
    dt_bias = torch.randn(channels, device=dev).requires_grad_()

    def scan_fwd():
        out[0] = selective_scan(x, dt, a, b, c, skip, z, dt_bias, None)

    ms = time_op(scan_fwd)
    nbytes = 4 * tokens * channels * 2
    exps = 2.0 * tokens * channels * state
    r = {"op": "selective_scan_fwd", "ms": ms, "gbs": nbytes / ms / 1e6, "frac_of_peak": nbytes / ms / 1e6 / hbm, "peak_kind": kind,
         "gexp_per_s": exps / ms / 1e6}
    results.append(r)
    print(json.dumps(r), flush=True)
    ms = time_op(lambda: torch.autograd.grad(out[0], (x, dt, a, b, c, skip, z, dt_bias), g, retain_graph=True))
    nbytes = 8 * tokens * channels * 2
    r = {"op": "selective_scan_bwd", "ms": ms, "gbs": nbytes / ms / 1e6, "frac_of_peak": nbytes / ms / 1e6 / hbm, "peak_kind": kind,
         "gexp_per_s": 1.5 * exps / ms / 1e6}
    results.append(r)
    print(json.dumps(r), flush=True)

    # gated DeltaNet recurrence (PyTorch ops: chunk-local work batched over all chunks, one small product per chunk sequential), 32 heads of 128
    from fast_llm_b200.ops.ssm import chunk_delta_rule

    heads, dk = 32, 128
    q, k, v = (torch.randn(tokens, heads, dk, device=dev).bfloat16().requires_grad_() for _ in range(3))
    log_decay = (-torch.rand(tokens, heads, device=dev) * 0.1).requires_grad_()
    beta = torch.rand(tokens, heads, device=dev).requires_grad_()
    go = torch.randn(tokens, heads, dk, device=dev).bfloat16()

    def gdn_fwd():
        out[0] = chunk_delta_rule(q, k, v, log_decay, beta, None, normalize_qk=True)

    ms = time_op(gdn_fwd, iters=5)
    flops = 2.0 * tokens * heads * dk * dk * 3  # state update, read and query per token (the recurrence itself)
    r = {"op": "gdn_chunk_delta_rule_fwd", "ms": ms, "tflops": flops / ms / 1e9, "peak_kind": kind, "note": "chunk-local part in PyTorch ops (cuBLAS batched matmuls), state recurrence in flb_delta_state_scan"}
    results.append(r)
    print(json.dumps(r), flush=True)
    ms = time_op(lambda: torch.autograd.grad(out[0], (q, k, v, log_decay, beta), go.to(out[0].dtype), retain_graph=True), iters=5)
    r = {"op": "gdn_chunk_delta_rule_bwd", "ms": ms, "tflops": 2 * flops / ms / 1e9, "peak_kind": kind, "note": "autograd through the batched chunk-local ops; adjoint recurrence in flb_delta_state_scan"}
    results.append(r)
    print(json.dumps(r), flush=True)

    # Kimi delta attention: the same recurrence with a decay per key channel (chunks of 32, pairwise decays kept per channel)
    log_decay_kda = (-torch.rand(tokens, heads, dk, device=dev) * 0.1).requires_grad_()

    def kda_fwd():
        out[0] = chunk_delta_rule(q, k, v, log_decay_kda, beta, None, normalize_qk=True)

    ms = time_op(kda_fwd, iters=3)
    r = {"op": "kda_chunk_delta_rule_fwd", "ms": ms, "tflops": flops / ms / 1e9, "peak_kind": kind, "note": "as above with per-channel decays"}
    results.append(r)
    print(json.dumps(r), flush=True)
    ms = time_op(lambda: torch.autograd.grad(out[0], (q, k, v, log_decay_kda, beta), go.to(out[0].dtype), retain_graph=True), iters=3)
    r = {"op": "kda_chunk_delta_rule_bwd", "ms": ms, "tflops": 2 * flops / ms / 1e9, "peak_kind": kind, "note": "autograd"}
    results.append(r)
    print(json.dumps(r), flush=True)


def profile_attention():
    """Small fixed workload for an ncu capture: two forward + backward launches of attention at the Mistral-7B shape."""
    from fast_llm_b200.ops.attention import attention_backward_native, attention_forward_native

    t, heads, kv, d, window = 8192, 32, 8, 128, 4096
    nq, nkv = heads * d, kv * d
    qkv = torch.randn(t, nq + 2 * nkv, device="cuda", dtype=torch.bfloat16)
    cu = torch.tensor([0, t], device="cuda", dtype=torch.int32)
    dout = torch.randn(t, nq, device="cuda", dtype=torch.bfloat16)
    dqkv = torch.empty_like(qkv)
    for _ in range(2):
        out, lse = attention_forward_native(qkv, 0, qkv, nq, nq + nkv, cu, cu, t, heads, kv, d, True, window, d**-0.5)
        attention_backward_native(qkv, 0, qkv, nq, nq + nkv, out, dout, lse, cu, cu, t, heads, kv, d, dqkv, dqkv, True, window, d**-0.5)
    torch.cuda.synchronize()
    print("profile_attention done")


def profile_gemm_shapes():
    """ncu workload: one launch each of the CTA-pair GEMM in four layouts / shapes of the Mistral-7B MLP."""
    from fast_llm_b200.ops.gemm import matmul_nn, matmul_nt

    t, h, f = 8192, 4096, 14336
    x = torch.randn(t, h, device="cuda", dtype=torch.bfloat16)
    w1 = torch.randn(2 * f, h, device="cuda", dtype=torch.bfloat16)
    dy1 = torch.randn(t, 2 * f, device="cuda", dtype=torch.bfloat16)
    w2 = torch.randn(f, h, device="cuda", dtype=torch.bfloat16)   # stored transposed: [ffn, hidden]
    a2 = torch.randn(t, f, device="cuda", dtype=torch.bfloat16)
    dy2 = torch.randn(t, h, device="cuda", dtype=torch.bfloat16)
    from fast_llm_b200.ops.gemm import matmul_tn

    grad1 = torch.zeros(2 * f, h, device="cuda", dtype=torch.float32)
    for _ in range(2):
        matmul_tn(dy1, x, out=grad1, accumulate=True)   # mlp1 wgrad [28672, 4096, 8192]  A, B MN-major, fp32 accumulate
        matmul_nt(x, w1)        # mlp1 fprop  [8192, 28672, 4096]  A, B K-major
        matmul_nn(dy1, w1)      # mlp1 dgrad  [8192, 4096, 28672]  B MN-major
        matmul_nn(a2, w2)       # mlp2 fprop  [8192, 4096, 14336]  B MN-major (transposed weight)
        matmul_nt(dy2, w2)      # mlp2 dgrad  [8192, 14336, 4096]  A, B K-major
    torch.cuda.synchronize()
    print("profile_gemm_shapes done")


def profile_gated():
    """ncu workload: three launches of the layer-1 GEMM with the gated activation in its epilogue, [8192, 4096] x [28672, 4096]^T
    (operands and outputs about 1 GB)."""
    from fast_llm_b200.ops.activation import ActivationType
    from fast_llm_b200.ops.gemm import matmul_nt_gated

    x = torch.randn(8192, 4096, device="cuda", dtype=torch.bfloat16)
    w1 = torch.randn(28672, 4096, device="cuda", dtype=torch.bfloat16) / 64
    for _ in range(3):
        matmul_nt_gated(x, w1, ActivationType.silu.code)
    torch.cuda.synchronize()
    print("profile_gated done")


def profile_elementwise():
    """ncu workload: two rounds of every memory-bound kernel of a dense step at [8192, 4096] (ffn 14336, vocabulary 32000), each
    operand larger than L2 together with its outputs, about 3 GB on the device."""
    from fast_llm_b200.ops.activation import ActivationType, act_bwd_native
    from fast_llm_b200.ops.cross_entropy import cross_entropy_forward_backward
    from fast_llm_b200.ops.normalization import _bwd_native, _fwd_native
    from fast_llm_b200.ops.rotary import rope_

    t, h, f = 8192, 4096, 14336
    x = torch.randn(t, h, device="cuda", dtype=torch.bfloat16)
    d = torch.randn(t, h, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(h, device="cuda", dtype=torch.bfloat16)
    gu = torch.randn(t, 2 * f, device="cuda", dtype=torch.bfloat16)
    go = torch.randn(t, f, device="cuda", dtype=torch.bfloat16)
    qkv = torch.randn(t, 6144, device="cuda", dtype=torch.bfloat16)
    ang = torch.arange(t, device="cuda", dtype=torch.float64)[:, None] * (10000.0 ** (-torch.arange(0, 128, 2, device="cuda", dtype=torch.float64) / 128))[None]
    table = torch.cat([ang.cos(), ang.sin()], -1).float().contiguous()
    logits = torch.randn(t, 32000, device="cuda", dtype=torch.bfloat16)
    labels = torch.randint(0, 32000, (t,), device="cuda")
    for _ in range(2):
        _, y, rstd, _ = _fwd_native(x, d, w, None, 1e-5, False, False)
        _bwd_native(y, x, w, None, rstd, None, d, False, False, True)
        act_bwd_native(go, gu, True, ActivationType.silu, True)
        rope_(qkv, table, None, 40, 128, 128)
        cross_entropy_forward_backward(logits, labels, 1.0, in_place=False)
    torch.cuda.synchronize()
    print("profile_elementwise done")


def profile_ssm():
    """ncu workload: two forward + backward passes of the selective scan (8192 x 4096 x 16) and of the gated DeltaNet
    delta rule (8192 tokens x 16 heads x 128), about 1.5 GB on the device."""
    from fast_llm_b200.ops.ssm import chunk_delta_rule, selective_scan

    tokens, channels, state, groups = 8192, 4096, 16, 32
    dev = "cuda"
    x = torch.randn(tokens, channels, device=dev).bfloat16().requires_grad_()
    dt = (torch.randn(tokens, channels, device=dev) - 1).bfloat16().requires_grad_()
    z = torch.randn(tokens, channels, device=dev).bfloat16().requires_grad_()
    a = (-torch.rand(channels, state, device=dev) - 0.1).requires_grad_()
    b = torch.randn(tokens, groups, state, device=dev).bfloat16().requires_grad_()
    c = torch.randn(tokens, channels // state, state, device=dev).bfloat16().requires_grad_()
    skip = torch.randn(channels, device=dev).requires_grad_()
    g = torch.randn(tokens, channels, device=dev).bfloat16()
    heads, dk = 16, 128
    q, k, v = (torch.randn(tokens, heads, dk, device=dev).bfloat16().requires_grad_() for _ in range(3))
    log_decay = (-torch.rand(tokens, heads, device=dev) * 0.1).requires_grad_()
    beta = torch.rand(tokens, heads, device=dev).requires_grad_()
    go = torch.randn(tokens, heads, dk, device=dev).bfloat16()
    for _ in range(2):
        y = selective_scan(x, dt, a, b, c, skip, z, None, None)
        torch.autograd.grad(y, (x, dt, a, b, c, skip, z), g)
        o = chunk_delta_rule(q, k, v, log_decay, beta, None)
        torch.autograd.grad(o, (q, k, v, log_decay, beta), go.to(o.dtype))
    torch.cuda.synchronize()
    print("profile_ssm done")


def profile_moe():
    """ncu workload: two forward + backward passes of a small dropless MoE layer (hidden 4096, 4 experts of FFN 4096, top-2,
    8192 tokens; about 1 GB on the device), so that the grouped GEMM launches can be captured."""
    import fast_llm_b200.models.auto  # noqa: F401
    from fast_llm_b200.layers.moe import MoEMLPConfig
    from fast_llm_b200.parallel.topology import DistributedConfig
    from fast_llm_b200.tensor import TensorDim

    tokens, hidden = 8192, 4096
    config = MoEMLPConfig.from_dict({"type": "moe", "experts": 4, "experts_per_token": 2, "intermediate_size": 4096, "gated": True,
                                     "activation": "silu", "add_linear_biases": False, "implementation": "dropless"})
    config.validate()
    dc = DistributedConfig.from_dict({"compute_dtype": "bf16", "seed": 0, "world_size": 1, "rank": 0, "local_world_size": 1})
    dc.validate()
    layer = config.get_layer(dc, TensorDim("hidden", hidden))
    layer.set_names("mlp.")
    layer = layer.materialize(device=torch.device("cuda"), dtype=torch.bfloat16)
    x = torch.randn(tokens, hidden, device="cuda", dtype=torch.bfloat16)
    g = torch.randn(tokens, hidden, device="cuda", dtype=torch.bfloat16)
    for _ in range(2):
        xi = x.detach().requires_grad_()
        layer.forward(xi, {"training": True}).backward(g)
    torch.cuda.synchronize()
    print("profile_moe done")


def profile_gemm():
    """Small fixed workload for an ncu capture: three launches of the fprop GEMM on operands larger than L2."""
    from fast_llm_b200.ops.gemm import matmul_nt

    t, k, n = 8192, 4096, 6144
    x = torch.randn(t, k, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(n, k, device="cuda", dtype=torch.bfloat16)
    for _ in range(3):
        matmul_nt(x, w)
    torch.cuda.synchronize()
    print("profile_gemm done")


def bench_tp_linear(results):
    """Sequence-parallel column- and row-parallel linears (forward + backward) and the all-gather + GEMM alone, per path:
    NCCL collectives around the GEMMs, the pull pipeline (peer-copy kernel + one GEMM per chunk) and the single-launch
    GEMM fed by the peers' pushes.  Run one process per GPU:
        python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m fast_llm_b200.tools.bench_kernels tp_linear
    Times are CUDA events on the launching stream, maximum over ranks."""
    import os

    from fast_llm_b200.ops.linear import linear
    from fast_llm_b200.parallel import fused_tp

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    device = torch.device("cuda", torch.cuda.current_device())
    torch.distributed.init_process_group("nccl", device_id=device)
    group = torch.distributed.group.WORLD
    tokens, hidden, ffn = 8192, 4096, 14336
    _, tflops_peak, kind = _peaks()
    generator = torch.Generator(device=device).manual_seed(1234 + rank)
    rows, cols = tokens // world, 2 * ffn // world
    x_shard = torch.randn(rows, hidden, device=device, dtype=torch.bfloat16, generator=generator)
    grad_shard = torch.randn(rows, hidden, device=device, dtype=torch.bfloat16, generator=generator)
    w1 = (torch.randn(cols, hidden, device=device, dtype=torch.bfloat16, generator=generator) * hidden**-0.5).requires_grad_()
    w2 = (torch.randn(cols, hidden, device=device, dtype=torch.bfloat16, generator=generator) * cols**-0.5).requires_grad_()

    def layer():
        x = x_shard.clone().requires_grad_()
        h = linear(x, w1, None, mode="output", group=group, sequence_parallel=True)
        y = linear(h, w2, None, transposed_weight=True, mode="input", group=group, sequence_parallel=True)
        y.backward(grad_shard)
        w1.grad = w2.grad = None

    def timed(fn, iters=10):
        for _ in range(3):
            fn()
        times = []
        for _ in range(iters):
            torch.cuda.synchronize()
            torch.distributed.barrier()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            fn()
            end.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(end))
        times.sort()
        t = torch.tensor([times[len(times) // 2]], device=device)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        return t.item()

    flops_layer = 3 * 2.0 * tokens * hidden * cols * 2  # two linears, forward + two backward GEMMs each, per rank
    flops_gather = 2.0 * tokens * hidden * cols
    out = {"op": "tp_linear", "world": world, "shape": [tokens, hidden, cols], "peak_kind": kind}
    out["nccl_ms"] = timed(layer)
    context = fused_tp.enable(group, device, tokens, hidden)
    for name, single in (("pull_pipeline", False), ("pushed_single_launch", True)):
        context.single_launch = single
        out[f"{name}_ms"] = timed(layer)
        out[f"{name}_gather_gemm_ms"] = timed(lambda: context.all_gather_matmul(x_shard, w1.detach(), False))
    # the pieces of the backward, each against its NCCL counterpart
    from fast_llm_b200.ops.gemm import matmul_nn, matmul_tn

    context.single_launch = True
    h_full = torch.randn(tokens, cols, device=device, dtype=torch.bfloat16, generator=generator)
    dw = torch.zeros(cols, hidden, device=device, dtype=torch.float32)
    out["fused_gemm_reduce_scatter_ms"] = timed(lambda: context.matmul_reduce_scatter(h_full, w2.detach(), True))
    scattered = torch.empty(rows, hidden, device=device, dtype=torch.bfloat16)

    def nccl_gemm_reduce_scatter():
        torch.distributed.reduce_scatter_tensor(scattered, matmul_nn(h_full, w2.detach()), group=group)

    out["nccl_gemm_reduce_scatter_ms"] = timed(nccl_gemm_reduce_scatter)
    out["gemm_only_ms"] = timed(lambda: matmul_nn(h_full, w2.detach()))
    out["fused_gather_wgrad_ms"] = timed(lambda: context.wgrad_from_gathered(h_full, context.finish_gather(context.start_gather(x_shard)), dw, True, False))
    gathered = torch.empty(tokens, hidden, device=device, dtype=torch.bfloat16)

    def nccl_gather_wgrad():
        torch.distributed.all_gather_into_tensor(gathered, x_shard, group=group)
        matmul_tn(h_full, gathered, out=dw, accumulate=True)

    out["nccl_gather_wgrad_ms"] = timed(nccl_gather_wgrad)
    out["wgrad_only_ms"] = timed(lambda: matmul_tn(h_full, gathered, out=dw, accumulate=True))

    def nccl_gather_gemm():
        from fast_llm_b200.ops.gemm import matmul_nt

        torch.distributed.all_gather_into_tensor(gathered, x_shard, group=group)
        matmul_nt(gathered, w1.detach())

    out["nccl_gather_gemm_ms"] = timed(nccl_gather_gemm)
    bound_ms = flops_layer / (tflops_peak * 1e9)
    out["compute_bound_ms"] = bound_ms
    out["gather_gemm_compute_bound_ms"] = flops_gather / (tflops_peak * 1e9)
    out["gather_bytes_per_rank"] = (world - 1) * rows * hidden * 2
    out["gather_link_bound_ms"] = out["gather_bytes_per_rank"] / 770e6  # measured peer copy, 770 GB/s per direction
    torch.cuda.synchronize()
    context.arena.check_errors()
    fused_tp.disable(group)
    if rank == 0:
        results.append(out)
        print(json.dumps(out), flush=True)
    torch.distributed.barrier()
    torch.distributed.destroy_process_group()


def bench_zero(results):
    """The two ZeRO kernels over NVLink peer memory in isolation: `flb_rs_reduce` (each rank sums its 1/n slice of every rank's
    fp32 gradient buffer with peer loads) and `flb_adam_push` (AdamW on the shard, bf16 weights stored into every rank's weight
    buffer), against NCCL's reduce-scatter / all-gather of the same buffers.  Run one process per GPU:
        python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m fast_llm_b200.tools.bench_kernels zero
    CUDA events, median of 10, maximum over ranks; rates are the bytes that cross NVLink per rank and direction."""
    import os

    from fast_llm_b200.parallel.symmetric import SymmetricArena, adam_push, rs_reduce

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    device = torch.device("cuda", torch.cuda.current_device())
    torch.distributed.init_process_group("nccl", device_id=device)
    group = torch.distributed.group.WORLD
    elements = 218 * 1024 * 1024  # one Mistral-7B decoder layer: 218 M parameters
    elements -= elements % (world * 8)
    shard = elements // world
    arena = SymmetricArena(elements * 4 + elements * 2, group, device)
    grads = arena.buffer[: elements * 4].view(torch.float32)
    weights = arena.buffer[elements * 4 :].view(torch.bfloat16)
    grads.normal_()
    grad_shard = torch.empty(shard, device=device)
    w, m, v = (torch.zeros(shard, device=device) for _ in range(3))
    lib = _lib_module().get_lib()
    partial = torch.empty(lib.flb_rs_reduce_blocks(), device=device)

    def timed(fn, iters=10):
        for _ in range(3):
            fn()
        times = []
        for _ in range(iters):
            torch.cuda.synchronize()
            torch.distributed.barrier()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            fn()
            end.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(end))
        times.sort()
        t = torch.tensor([times[len(times) // 2]], device=device)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        return t.item()

    def fused_reduce():
        arena.barrier(0)
        rs_reduce(arena, grads, grad_shard, shard, 1.0 / world, False, partial)
        arena.barrier(0)

    def fused_update():
        adam_push(arena, w, grad_shard, m, v, weights[rank * shard : (rank + 1) * shard], 1e-4, 0.9, 0.95, 1e-8, 0.1, 1, None)
        arena.barrier(1)

    gathered = torch.empty(elements, dtype=torch.bfloat16, device=device)
    low = torch.empty(shard, dtype=torch.bfloat16, device=device)
    out = {"op": "zero_kernels", "world": world, "elements": elements}
    out["rs_reduce_ms"] = timed(fused_reduce)
    if arena.multicast_ptr:
        # the same reduction with the sums formed inside NVSwitch (multimem.ld_reduce): one pull of the slice instead of one per peer
        rank_ordered = grad_shard.clone()
        os.environ["FLB_ZERO_MULTIMEM"] = "1"
        out["rs_reduce_multimem_ms"] = timed(fused_reduce)
        out["rs_reduce_multimem_max_abs_difference"] = (grad_shard - rank_ordered).abs().max().item()
        os.environ["FLB_ZERO_MULTIMEM"] = "0"
    else:
        out["rs_reduce_multimem_ms"] = None  # no multicast mapping on this fabric / driver
    out["nccl_reduce_scatter_ms"] = timed(lambda: torch.distributed.reduce_scatter_tensor(grad_shard, grads, group=group))
    out["adam_push_ms"] = timed(fused_update)
    out["nccl_all_gather_ms"] = timed(lambda: torch.distributed.all_gather_into_tensor(gathered, low, group=group))
    pulled = (world - 1) * shard * 4  # fp32 gradient slices read from the peers
    pushed = (world - 1) * shard * 2  # bf16 weights stored into the peers
    out["rs_reduce_nvlink_gbs"] = pulled / out["rs_reduce_ms"] / 1e6
    out["adam_push_nvlink_gbs"] = pushed / out["adam_push_ms"] / 1e6
    out["rs_reduce_link_bound_ms"] = pulled / 770e6
    out["adam_push_link_bound_ms"] = pushed / 770e6
    out["adam_push_hbm_bound_ms"] = shard * 30 / (_peaks()[0] * 1e6)  # 28 bytes per element locally + the local bf16 copy
    torch.cuda.synchronize()
    arena.check_errors()
    if rank == 0:
        results.append(out)
        print(json.dumps(out), flush=True)
    torch.distributed.barrier()
    torch.distributed.destroy_process_group()


def bench_generate(results):
    """Greedy generation through the Hugging Face wrapper with and without the key / value cache (one GPU): a decoder of
    8 blocks, hidden 2048, 16 heads of 128 (4 groups), vocabulary 32000; 8 prompts of 512 tokens, 32 new tokens each."""
    import fast_llm_b200.models.auto  # noqa: F401
    from fast_llm_b200.engine.inference.huggingface import HuggingfaceGPTModelForCausalLM
    from fast_llm_b200.engine.multi_stage.config import StageMode
    from fast_llm_b200.models.gpt.config import GPTModelConfig
    from fast_llm_b200.models.gpt.model import GPTModel
    from fast_llm_b200.parallel.distributed import Distributed

    config = GPTModelConfig.from_dict({
        "base_model": {
            "embeddings": {"vocab_size": 32000}, "hidden_size": 2048,
            "decoder": {"num_blocks": 8, "block": {
                "mixer": {"type": "attention", "rotary": {"type": "default"}, "heads": 16, "head_groups": 4, "head_size": 128, "add_linear_biases": False},
                "mlp": {"intermediate_size": 8192, "gated": True, "activation": "silu", "add_linear_biases": False},
                "normalization": {"type": "rms_norm"}}},
            "head": {"normalization": {"type": "rms_norm"}}},
        "distributed": {"compute_dtype": "bf16", "world_size": 1, "rank": 0, "local_world_size": 1}})
    config.validate()
    model = GPTModel(config)
    model.setup(Distributed(config.distributed), mode=StageMode.inference)
    model.initialize_weights()
    wrapper = HuggingfaceGPTModelForCausalLM(model)
    torch.manual_seed(0)
    rows, prompt_length, new_tokens = 8, 512, 32
    prompt = torch.randint(1, 32000, (rows, prompt_length), device="cuda")
    mask = torch.ones_like(prompt)
    for use_cache in (True, False):
        arguments = dict(attention_mask=mask, max_new_tokens=new_tokens, min_new_tokens=new_tokens, do_sample=False, pad_token_id=0, use_cache=use_cache)
        wrapper.generate(prompt, **{**arguments, "max_new_tokens": 4, "min_new_tokens": 4})  # warm-up
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        out = wrapper.generate(prompt, **arguments)
        end.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(end)
        assert out.shape == (rows, prompt_length + new_tokens)
        entry = {"name": f"generate_{'cached' if use_cache else 'uncached'}", "ms": ms, "new_tokens_per_s": rows * new_tokens / ms * 1e3}
        results.append(entry)
        print(f"generate use_cache={use_cache}: {ms:9.1f} ms for {rows} x {new_tokens} new tokens after {prompt_length}: {entry['new_tokens_per_s']:8.1f} tokens/s")
    from fast_llm_b200.utils.device_errors import check_device_errors

    check_device_errors()
    return results


def _lib_module():
    from fast_llm_b200.ops import _lib

    return _lib


def main(argv):
    results = []
    if "tp_linear" in argv:
        return bench_tp_linear(results)
    if "zero" in argv:
        return bench_zero(results)
    if "generate" in argv:
        return bench_generate(results)
    if "profile_gemm" in argv:
        return profile_gemm()
    if "profile_gemm_shapes" in argv:
        return profile_gemm_shapes()
    if "profile_attention" in argv:
        return profile_attention()
    if "profile_ssm" in argv:
        return profile_ssm()
    if "profile_elementwise" in argv:
        return profile_elementwise()
    if "profile_gated" in argv:
        return profile_gated()
    if "profile_moe" in argv:
        return profile_moe()
    if "gemm_tiles" in argv:
        bench_gemm_tiles(results)
    if "attention" in argv:
        bench_attention(results)
    if "moe" in argv:
        bench_moe(results)
    if "ssm" in argv:
        bench_ssm(results)
    which = [a for a in argv if a in ("gemm", "elementwise")] or ([] if ("gemm_tiles" in argv or "attention" in argv or "moe" in argv or "ssm" in argv) else ["gemm", "elementwise"])
    if "gemm" in which:
        bench_gemm(results)
    if "elementwise" in which:
        bench_elementwise(results)
    if "--json" in argv:
        pathlib.Path(argv[argv.index("--json") + 1]).write_text(json.dumps(results, indent=1))


if __name__ == "__main__":
    main(sys.argv[1:])
