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
