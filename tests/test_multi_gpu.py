"""Multi-GPU paths (NCCL + the fused peer-memory ZeRO kernels).  Needs at least 2 GPUs; skipped otherwise."""

import pytest
import torch

from tests.distributed_utils import run_distributed

pytestmark = pytest.mark.gpu


def _gpu_rank_main(rank, world_size, updates, steps):
    import torch

    from tests.common import build_trainer, tiny_trainer_config, train_steps

    torch.cuda.set_device(rank)
    updates = {("model", "distributed", "use_cuda"): True, ("model", "distributed", "compute_dtype"): "bf16",
               ("model", "distributed", "world_size"): world_size, ("model", "distributed", "rank"): rank,
               ("model", "distributed", "local_world_size"): world_size, ("model", "distributed", "reproducible_init"): True,
               ("data", "micro_batch_size"): 512, **updates}
    trainer, distributed = build_trainer(tiny_trainer_config(updates))
    fused = trainer.multi_stage.weight_arena is not None
    losses = train_steps(trainer, steps)
    torch.cuda.synchronize()
    if fused:
        trainer.multi_stage.weight_arena.check_errors()
        trainer.multi_stage.grad_arena.check_errors()
    weights = {n: t.float().cpu().numpy() for n, _, t in trainer.multi_stage.get_state_tensor_iterator(("weights",))}
    # the bf16 weight buffers every rank computes with must equal the rounded master weights of their owners
    trainer.multi_stage.invalidate_buffers() if not fused else None
    buffers = {}
    for stage in trainer.multi_stage.stages_on_device.values():
        if not fused:
            stage.restore_parameters()
        for name in stage.parameter_names:
            buffers[name] = stage.get_parameter_meta(name).tensor.detach().float().cpu().numpy()
    distributed.shutdown()
    return losses, weights, buffers, fused


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_zero_matches_nccl_path():
    steps = 3
    base = {("schedule", "depth_first_micro_batches"): 2}
    fused = run_distributed(_gpu_rank_main, 2, base, steps, timeout=600)
    plain = run_distributed(_gpu_rank_main, 2, {**base, ("model", "multi_stage", "fused_collectives"): False}, steps, timeout=600)
    assert all(r[3] for r in fused), "fused path was not active (symmetric memory unavailable?)"
    assert not any(r[3] for r in plain)
    for (lf, wf, bf, _), (lp, wp, bp, _) in zip(fused, plain):
        assert lf == pytest.approx(lp, rel=2e-3)
        for name in wp:
            torch.testing.assert_close(torch.from_numpy(wf[name]), torch.from_numpy(wp[name]), rtol=1e-3, atol=4e-3, msg=lambda m: f"{name}: {m}")  # Adam steps are ~lr each; atomics reorder tiny gradients
            torch.testing.assert_close(torch.from_numpy(bf[name]), torch.from_numpy(bp[name]), rtol=1e-2, atol=1e-3, msg=lambda m: f"buffer {name}: {m}")
    # both ranks hold identical weights and buffers
    for name in fused[0][1]:
        assert (fused[0][1][name] == fused[1][1][name]).all()
        assert (fused[0][2][name] == fused[1][2][name]).all(), name


def _gradient_rank_main(rank, world_size, updates):
    """One step without the optimizer: this rank's reduced fp32 gradient shards and the global gradient norm."""
    import torch

    from tests.common import build_trainer, tiny_trainer_config, train_steps
    from fast_llm_b200.engine.multi_stage.multi_stage import ShardName

    torch.cuda.set_device(rank)
    updates = {("model", "distributed", "use_cuda"): True, ("model", "distributed", "compute_dtype"): "bf16",
               ("model", "distributed", "world_size"): world_size, ("model", "distributed", "rank"): rank,
               ("model", "distributed", "local_world_size"): world_size, ("model", "distributed", "reproducible_init"): True,
               ("data", "micro_batch_size"): 512, ("schedule", "depth_first_micro_batches"): 2, **updates}
    trainer, distributed = build_trainer(tiny_trainer_config(updates))
    fused = trainer.multi_stage.weight_arena is not None
    from fast_llm_b200.parallel.topology import PhaseType

    schedule = trainer._schedules[PhaseType.training]
    iterator = trainer._data.get_iterator("training", consumed_samples=0, num_workers=0)
    losses, ok, metrics = trainer.runner.run_step(iterator, schedule, iteration=1, return_metrics=True)
    torch.cuda.synchronize()
    from fast_llm_b200.utils.device_errors import check_device_errors

    check_device_errors(distributed.world_group, distributed.device)
    grads = trainer.multi_stage._shards[ShardName.grads].float().cpu().numpy()
    norm = float(metrics["grad_norm"])
    distributed.shutdown()
    return losses, grads, norm, fused


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_reduction_gives_the_same_gradient_shards_and_norm_as_nccl():
    """The reduced fp32 gradient shards themselves (not weights after Adam, where a step is about one learning rate whatever
    the gradient): peer-load reduction in rank order against NCCL's reduce-scatter, and the norm finished from the kernel's
    per-block partial sums against the separate norm pass.  The embedding backward adds rows with atomics, so the last bits of
    its gradient depend on the order of arrival: tolerance 1e-5 relative."""
    fused = run_distributed(_gradient_rank_main, 2, {("optimizer", "learning_rate", "base"): 0.0}, timeout=600)
    plain = run_distributed(_gradient_rank_main, 2, {("optimizer", "learning_rate", "base"): 0.0, ("model", "multi_stage", "fused_collectives"): False},
                            timeout=600)
    assert all(r[3] for r in fused) and not any(r[3] for r in plain)
    for (lf, gf, nf, _), (lp, gp, np_, _) in zip(fused, plain):
        assert lf == pytest.approx(lp, rel=1e-6)
        torch.testing.assert_close(torch.from_numpy(gf), torch.from_numpy(gp), rtol=1e-5, atol=1e-8)
        assert nf == pytest.approx(np_, rel=1e-5)
    assert fused[0][2] == fused[1][2], "every rank computes the same global norm"


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("name,updates", [
    ("zero2", {("model", "multi_stage", "zero_stage"): 2}),
    ("zero3", {("model", "multi_stage", "zero_stage"): 3}),
    ("zero3_two_buffers", {("model", "multi_stage", "zero_stage"): 3, ("model", "multi_stage", "num_weight_buffers"): 2,
                           ("model", "multi_stage", "num_grad_buffers"): 2}),
])
def test_zero_stages_on_gpus_match_stage_one(name, updates):
    """ZeRO-2 / ZeRO-3 on real streams: weight gathers issued one step ahead into buffers shared round-robin between stages,
    gradient buffers reused after their reduction - the events that guard them are only exercised on a GPU."""
    steps = 3
    base = {("schedule", "depth_first_micro_batches"): 2, ("model", "multi_stage", "fused_collectives"): False}
    reference = run_distributed(_gpu_rank_main, 2, base, steps, timeout=600)
    sharded = run_distributed(_gpu_rank_main, 2, {**base, **updates}, steps, timeout=600)
    for (lr_, wr, _, _), (ls, ws, _, _) in zip(reference, sharded):
        assert ls == pytest.approx(lr_, rel=2e-3), name
        for key in wr:
            torch.testing.assert_close(torch.from_numpy(ws[key]), torch.from_numpy(wr[key]), rtol=1e-3, atol=4e-3, msg=lambda m: f"{name} {key}: {m}")


def _pipeline_rank_main(rank, world_size, updates, steps):
    import torch

    from tests.common import build_trainer, tiny_trainer_config, train_steps

    torch.cuda.set_device(rank)
    updates = {("model", "distributed", "use_cuda"): True, ("model", "distributed", "compute_dtype"): "bf16",
               ("model", "distributed", "world_size"): world_size, ("model", "distributed", "rank"): rank,
               ("model", "distributed", "local_world_size"): world_size, ("model", "distributed", "reproducible_init"): True,
               ("data", "micro_batch_size"): 512, **updates}
    trainer, distributed = build_trainer(tiny_trainer_config(updates))
    losses = train_steps(trainer, steps)
    torch.cuda.synchronize()
    distributed.shutdown()
    return losses


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("tied", [False, True])
def test_pipeline_parallel_on_gpus_matches_one_gpu(tied):
    """Two pipeline ranks over NCCL point-to-point with the receives posted early in the common transfer order (four
    micro-batches in flight, so every rank has sends and receives interleaved): same losses as the whole model on one GPU."""
    steps = 3
    common = {("schedule", "breadth_first_micro_batches"): 4, ("model", "base_model", "tied_embedding_weight"): tied}
    single = run_distributed(_pipeline_rank_main, 1, common, steps, timeout=600)[0]
    piped = run_distributed(_pipeline_rank_main, 2, {**common, ("model", "distributed", "pipeline_parallel"): 2}, steps, timeout=600)
    for losses in piped:
        assert losses == pytest.approx(single, rel=5e-3)


def _fused_tp_rank_main(rank, world_size, tokens, hidden, ffn, timing):
    """Sequence-parallel column- and row-parallel linears, forward and backward: fused peer-memory kernels vs NCCL."""
    import torch

    from fast_llm_b200.ops.activation import ActivationType
    from fast_llm_b200.ops.linear import linear
    from fast_llm_b200.ops.mlp import MLPRecomputeLevel, mlp
    from fast_llm_b200.parallel import fused_tp

    torch.cuda.set_device(rank)
    torch.distributed.init_process_group("nccl", rank=rank, world_size=world_size, device_id=torch.device("cuda", rank))
    group = torch.distributed.group.WORLD
    device = torch.device("cuda", rank)
    generator = torch.Generator(device=device).manual_seed(1234)  # same weights / activations layout on all ranks
    full_x = torch.randn(tokens, hidden, device=device, dtype=torch.bfloat16, generator=generator)
    w_out_full = torch.randn(ffn, hidden, device=device, dtype=torch.bfloat16, generator=generator) * hidden**-0.5
    w_in_full = torch.randn(ffn, hidden, device=device, dtype=torch.bfloat16, generator=generator) * ffn**-0.5  # stored [in, out]
    grad_full = torch.randn(tokens, hidden, device=device, dtype=torch.bfloat16, generator=generator)
    rows, cols = tokens // world_size, ffn // world_size
    x_shard = full_x[rank * rows : (rank + 1) * rows].clone()
    grad_shard = grad_full[rank * rows : (rank + 1) * rows].clone()

    def run():
        x = x_shard.clone().requires_grad_()
        w1 = w_out_full[rank * cols : (rank + 1) * cols].clone().requires_grad_()
        w2 = w_in_full[rank * cols : (rank + 1) * cols].clone().requires_grad_()
        h = linear(x, w1, None, mode="output", group=group, sequence_parallel=True)          # [T, ffn/tp]
        y = linear(h, w2, None, transposed_weight=True, mode="input", group=group, sequence_parallel=True)  # [T/tp, hidden]
        y.backward(grad_shard)
        outputs = [t.detach().float() for t in (h, y, x.grad, w1.grad, w2.grad)]
        # the MLP node: gated layer 1 (gate rows, then up rows, of this rank's slice), layer 2 stored [ffn/tp, hidden]
        xm = x_shard.clone().requires_grad_()
        half = cols // 2
        m1 = torch.cat([w_out_full[rank * half : (rank + 1) * half], w_out_full[ffn // 2 + rank * half : ffn // 2 + (rank + 1) * half]]).clone().requires_grad_()
        m2 = w_in_full[rank * half : (rank + 1) * half].clone().requires_grad_()
        out = mlp(xm, m1, None, m2, None, gated=True, activation=ActivationType.silu, group=group, sequence_parallel=True,
                  recompute_level=MLPRecomputeLevel.activation)
        out.backward(grad_shard)
        return outputs + [t.detach().float() for t in (out, xm.grad, m1.grad, m2.grad)]

    def time_it():
        for _ in range(3):
            run()
        torch.cuda.synchronize()
        torch.distributed.barrier()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(10):
            run()
        end.record()
        torch.cuda.synchronize()
        elapsed = torch.tensor([start.elapsed_time(end) / 10], device=device)
        torch.distributed.all_reduce(elapsed, op=torch.distributed.ReduceOp.MAX)
        return elapsed.item()

    plain = run()
    plain_ms = time_it() if timing else None
    context = fused_tp.enable(group, device, tokens, max(hidden, 8))
    fused = run()
    fused_again = run()  # exercises the double buffering
    fused_ms = time_it() if timing else None
    torch.cuda.synchronize()
    context.arena.check_errors()
    from fast_llm_b200.ops.gemm import check_device_errors

    check_device_errors()
    errors = []
    for a, b, c in zip(plain, fused, fused_again):
        scale = a.abs().mean().item() + 1e-6
        errors.append(((a - b).abs().max().item() / scale, (b - c).abs().max().item()))
    fused_tp.disable(group)
    torch.distributed.barrier()
    return errors, plain_ms, fused_ms


def _pushed_gather_rank_main(rank, world_size, shapes, repeats):
    """`all_gather_matmul` as one GEMM launch fed by the peers' pushes, against an NCCL all-gather followed by the same GEMM."""
    import torch

    from fast_llm_b200.ops.gemm import check_device_errors, matmul_nn, matmul_nt
    from fast_llm_b200.parallel import fused_tp

    torch.cuda.set_device(rank)
    torch.distributed.init_process_group("nccl", rank=rank, world_size=world_size, device_id=torch.device("cuda", rank))
    group = torch.distributed.group.WORLD
    device = torch.device("cuda", rank)
    max_tokens = max(rows for rows, _, _ in shapes) * world_size
    context = fused_tp.enable(group, device, max_tokens, max(k for _, k, _ in shapes))
    assert context.single_launch
    worst = 0.0
    for repeat in range(repeats):
        for index, (rows, k, n) in enumerate(shapes):
            generator = torch.Generator(device=device).manual_seed(100 * repeat + index)
            full = torch.randn(rows * world_size, k, device=device, dtype=torch.bfloat16, generator=generator)
            b_mn = (repeat + index) % 2 == 1
            weight = torch.randn((k, n) if b_mn else (n, k), device=device, dtype=torch.bfloat16, generator=generator) * k**-0.5
            shard = full[rank * rows : (rank + 1) * rows].clone()
            out = context.all_gather_matmul(shard, weight, b_mn)
            shard.zero_()  # the caller may reuse its shard at once
            gathered = torch.empty_like(full)
            torch.distributed.all_gather_into_tensor(gathered, full[rank * rows : (rank + 1) * rows].contiguous())
            reference = matmul_nn(gathered, weight) if b_mn else matmul_nt(gathered, weight)
            worst = max(worst, (out.float() - reference.float()).abs().max().item())
    torch.cuda.synchronize()
    context.arena.check_errors()
    check_device_errors()
    fused_tp.disable(group)
    torch.distributed.barrier()
    return worst


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_pushed_all_gather_matmul_is_the_gathered_gemm_bit_for_bit():
    # shard rows that are and are not multiples of the 256-row tile; calls alternate landing halves and weight layouts
    shapes = [(512, 256, 384), (328, 192, 520), (1024, 512, 1024), (72, 64, 136)]
    assert run_distributed(_pushed_gather_rank_main, 2, shapes, 3, timeout=600) == [0.0, 0.0]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_tensor_parallel_linear_matches_nccl():
    results = run_distributed(_fused_tp_rank_main, 2, 1024, 512, 1536, False, timeout=600)
    for errors, _, _ in results:
        for relative, repeat in errors:
            assert relative < 0.15, errors  # bf16 partial sums are rounded once more on the fused path
            assert repeat == 0.0, errors  # deterministic


def _fused_ce_rank_main(rank, world_size, rows, vocab):
    import torch

    from fast_llm_b200.ops.cross_entropy import cross_entropy_forward_backward, cross_entropy_reference
    from fast_llm_b200.parallel import fused_ce

    torch.cuda.set_device(rank)
    torch.distributed.init_process_group("nccl", rank=rank, world_size=world_size, device_id=torch.device("cuda", rank))
    group = torch.distributed.group.WORLD
    torch.manual_seed(0)
    full = (torch.randn(rows, vocab, device="cuda") * 3).bfloat16()
    labels = torch.randint(0, vocab, (rows,), device="cuda")
    labels[::7] = -100
    shard = vocab // world_size
    local = full[:, rank * shard : (rank + 1) * shard].contiguous()
    reference = cross_entropy_reference(full.float(), labels, 0.5, 1.0, 1e-4)
    plain = cross_entropy_forward_backward(local.clone(), labels, 0.5, 1.0, 1e-4, group, rank * shard)
    context = fused_ce.enable(group, torch.device("cuda", rank))
    results = []
    for _ in range(3):  # both halves of the double buffer, and reuse
        results.append(cross_entropy_forward_backward(local.clone(), labels, 0.5, 1.0, 1e-4, group, rank * shard))
    torch.cuda.synchronize()
    context._arena.check_errors()
    fused_ce.disable(group)
    out = []
    for loss, z, grad in results:
        out.append((float((loss - plain[0]).abs().max()), float((z - plain[1]).abs().max()), float((grad.float() - plain[2].float()).abs().max()),
                    float((loss - reference[0]).abs().max()),
                    float((grad.float() - reference[2][:, rank * shard : (rank + 1) * shard]).abs().max())))
    torch.distributed.barrier()
    torch.distributed.destroy_process_group()
    return out


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_cross_entropy_exchange_matches_all_reduce():
    for per_rank in run_distributed(_fused_ce_rank_main, 2, 777, 4096, timeout=600):
        for d_loss, d_z, d_grad, d_loss_ref, d_grad_ref in per_rank:
            assert d_loss < 1e-4 and d_z < 1e-2 and d_grad < 1e-3, per_rank
            assert d_loss_ref < 2e-2 and d_grad_ref < 2e-2, per_rank


def _tp_training_rank_main(rank, world_size, updates, steps):
    import torch

    from fast_llm_b200.parallel import fused_ce, fused_tp
    from tests.common import build_trainer, tiny_trainer_config, train_steps

    torch.cuda.set_device(rank)
    updates = {("model", "distributed", "use_cuda"): True, ("model", "distributed", "compute_dtype"): "bf16",
               ("model", "distributed", "world_size"): world_size, ("model", "distributed", "rank"): rank,
               ("model", "distributed", "local_world_size"): world_size, ("model", "distributed", "reproducible_init"): True,
               ("model", "distributed", "tensor_parallel"): world_size, ("model", "distributed", "sequence_tensor_parallel"): True,
               ("data", "micro_batch_size"): 512, **updates}
    trainer, distributed = build_trainer(tiny_trainer_config(updates))
    losses = train_steps(trainer, steps)
    torch.cuda.synchronize()
    group = distributed.tensor_group
    linear_context, loss_context = fused_tp.get(group), fused_ce.get(group)
    used = (linear_context is not None and linear_context.max_tokens is not None, loss_context is not None and loss_context._arena is not None)
    for context in (linear_context, loss_context):
        arena = getattr(context, "arena", None) or getattr(context, "_arena", None)
        if arena is not None:
            arena.check_errors()
    distributed.shutdown()
    return losses, used


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tensor_parallel_training_with_fused_collectives():
    """Two tensor-parallel ranks (sequence-parallel): GEMMs fused with their collectives and the loss statistics exchange
    over peer memory give the losses of the NCCL path."""
    steps = 3
    fused = run_distributed(_tp_training_rank_main, 2, {}, steps, timeout=600)
    plain = run_distributed(_tp_training_rank_main, 2, {("model", "multi_stage", "fused_collectives"): False}, steps, timeout=600)
    assert all(r[1] == (True, True) for r in fused), [r[1] for r in fused]
    assert all(r[1] == (False, False) for r in plain), [r[1] for r in plain]
    for (lf, _), (lp, _) in zip(fused, plain):
        assert lf == pytest.approx(lp, rel=2e-2)
    assert fused[0][0] == pytest.approx(fused[1][0], rel=1e-6)


def _sdp_training_rank_main(rank, world_size, updates, steps):
    import torch

    from fast_llm_b200.parallel import fused_sdp
    from tests.common import build_trainer, tiny_trainer_config, train_steps

    torch.cuda.set_device(rank)
    updates = {("model", "distributed", "use_cuda"): True, ("model", "distributed", "compute_dtype"): "bf16",
               ("model", "distributed", "world_size"): world_size, ("model", "distributed", "rank"): rank,
               ("model", "distributed", "local_world_size"): world_size, ("model", "distributed", "reproducible_init"): True,
               ("model", "distributed", "sequence_data_parallel"): world_size, ("data", "micro_batch_size"): 512, **updates}
    trainer, distributed = build_trainer(tiny_trainer_config(updates))
    losses = train_steps(trainer, steps)
    torch.cuda.synchronize()
    context = fused_sdp.get(distributed.sequence_data_group)
    used = context is not None and context.arena is not None and context._gathers > 0 and context._scatters > 0
    if context is not None and context.arena is not None:
        context.arena.check_errors()
    distributed.shutdown()
    return losses, used


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_sequence_data_parallel_exchange_through_symmetric_memory():
    steps = 3
    fused = run_distributed(_sdp_training_rank_main, 2, {}, steps, timeout=600)
    plain = run_distributed(_sdp_training_rank_main, 2, {("model", "multi_stage", "fused_collectives"): False}, steps, timeout=600)
    assert all(r[1] for r in fused) and not any(r[1] for r in plain)
    for (lf, _), (lp, _) in zip(fused, plain):
        assert lf == pytest.approx(lp, rel=1e-2)


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs 4 GPUs")
def test_fused_collectives_on_four_ranks():
    """The peer-memory kernels at group size 4: tensor-parallel linears and the loss-statistics exchange."""
    results = run_distributed(_fused_tp_rank_main, 4, 2048, 512, 2048, False, timeout=600)
    for errors, _, _ in results:
        for relative, repeat in errors:
            assert relative < 0.15, errors
            assert repeat == 0.0, errors
    assert run_distributed(_pushed_gather_rank_main, 4, [(512, 256, 384), (200, 192, 520), (768, 512, 1024)], 3, timeout=600) == [0.0] * 4
    for per_rank in run_distributed(_fused_ce_rank_main, 4, 515, 8192, timeout=600):
        for d_loss, d_z, d_grad, d_loss_ref, d_grad_ref in per_rank:
            assert d_loss < 1e-4 and d_z < 1e-2 and d_grad < 1e-3, per_rank
            assert d_loss_ref < 2e-2 and d_grad_ref < 2e-2, per_rank


def _multimem_rank_main(rank, world_size):
    import os

    import torch

    from fast_llm_b200.parallel.symmetric import SymmetricArena, rs_reduce

    torch.cuda.set_device(rank)
    torch.distributed.init_process_group("nccl", rank=rank, world_size=world_size, device_id=torch.device("cuda", rank))
    device = torch.device("cuda", rank)
    elements = 8 * 1024 * 1024
    shard = elements // world_size
    arena = SymmetricArena(elements * 4, torch.distributed.group.WORLD, device)
    grads = arena.buffer.view(torch.float32)
    grads.copy_(torch.randn(elements, device=device, generator=torch.Generator(device=device).manual_seed(rank)))
    outputs = []
    for flag in ("0", "1"):
        os.environ["FLB_ZERO_MULTIMEM"] = flag
        out = torch.zeros(shard, device=device)
        arena.barrier(0)
        rs_reduce(arena, grads, out, shard, 1.0 / world_size, False, None)
        arena.barrier(0)
        outputs.append(out)
    os.environ["FLB_ZERO_MULTIMEM"] = "0"
    torch.cuda.synchronize()
    arena.check_errors()
    result = (bool(arena.multicast_ptr), (outputs[0] - outputs[1]).abs().max().item(), outputs[0].abs().max().item())
    torch.distributed.barrier()
    return result


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_in_switch_gradient_reduction_agrees_with_the_rank_ordered_kernel():
    """`FLB_ZERO_MULTIMEM=1`: the slice sums come from `multimem.ld_reduce` (one pull through NVSwitch); same values as the
    peer-load kernel up to the order of the fp32 additions.  Without a multicast mapping the option changes nothing."""
    for available, difference, magnitude in run_distributed(_multimem_rank_main, 2, timeout=600):
        assert magnitude > 0.1
        assert difference <= (1e-6 * magnitude if available else 0.0) + 1e-7
