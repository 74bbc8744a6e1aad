"""Language-model losses: values and logit gradients against fp32 autograd restatements, against the reference's own
PyTorch functions where that tree is present, over 1 and 2 vocabulary shards (Gloo), with and without a loss mask.
Model of the cases: `tests/layers/test_lm_losses.py:1103-1634` of the reference."""

import os
import pathlib
import sys

import pytest
import torch

from tests.distributed_utils import run_distributed

# the reference checkout: $FAST_LLM_REFERENCE, else a `reference` directory beside this repository
REFERENCE = pathlib.Path(os.environ.get("FAST_LLM_REFERENCE") or pathlib.Path(__file__).resolve().parents[2] / "reference")
T, V = 48, 96


def _inputs(seed=0, mask_some=True):
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(T, V, generator=g) * 2
    teacher = torch.randn(T, V, generator=g) * 2
    labels = torch.randint(0, V, (T,), generator=g)
    if mask_some:
        labels[torch.rand(T, generator=g) < 0.25] = -100
    advantages = torch.randn(T, generator=g)
    old = -torch.rand(T, generator=g) * 3
    document = torch.sort(torch.randint(0, 5, (T,), generator=g)).values
    return logits, teacher, labels, advantages, old, document


# ---------------------------------------------------------------------------------------------------------------------
# fp32 autograd restatements (the oracle for every path of the library)
def _oracle_label(kind, logits, labels, scale, adv=None, old=None, doc=None, eps=(0.2, 0.2)):
    x = (logits.double() * scale).requires_grad_()
    lp = torch.log_softmax(x, -1)
    valid = labels >= 0
    count = valid.sum().clamp(min=1)
    picked = lp.gather(-1, labels.clamp(min=0)[:, None])[:, 0]
    if kind == "cross_entropy":
        loss = -(picked * valid).sum() / count
    elif kind == "z_loss":
        loss = ((torch.logsumexp(x, -1) ** 2) * valid).sum() / count
    elif kind == "grpo":
        ratio = torch.exp((picked - old) * valid)
        per = -torch.minimum(ratio * adv, ratio.clamp(1 - eps[0], 1 + eps[1]) * adv)
        loss = (per * valid).sum() / count
    elif kind == "gspo":
        n = int(doc.max()) + 1
        v = valid.double()
        num = torch.zeros(n, dtype=torch.double).index_add(0, doc, (picked - old) * v)
        den = torch.zeros(n, dtype=torch.double).index_add(0, doc, v)
        a = torch.zeros(n, dtype=torch.double).index_add(0, doc, adv.double() * v) / den.clamp(min=1)
        r = torch.exp(num / den.clamp(min=1))
        loss = (den * -torch.minimum(r * a, r.clamp(1 - eps[0], 1 + eps[1]) * a)).sum() / count
    else:
        raise NotImplementedError(kind)
    (grad,) = torch.autograd.grad(loss, x)
    return loss.float(), (grad * scale).float()


def _oracle_distribution(kind, logits, teacher, mask, scale, temperature):
    x = (logits.double() * scale).requires_grad_()  # the temperature softens the teacher only
    t = teacher.double() * (scale / temperature)
    lp, lq = torch.log_softmax(x, -1), torch.log_softmax(t, -1)
    if kind == "cross_entropy":
        per = -(lq.exp() * lp).sum(-1)
    elif kind == "forward_kl":
        per = (lq.exp() * (lq - lp)).sum(-1)
    else:
        per = (lp.exp() * (lp - lq)).sum(-1)
    m = torch.ones(T, dtype=torch.double) if mask is None else mask.double()
    loss = (per * m).sum() / m.sum().clamp(min=1)
    (grad,) = torch.autograd.grad(loss, x)
    return loss.float(), (grad * scale).float()


# ---------------------------------------------------------------------------------------------------------------------
class _Distributed:
    tensor_group = None
    sequence_data_group = None


def _layer(type_name, fields=None, group=None, vocab_begin=0):
    import fast_llm_b200.models.auto  # noqa: F401
    from fast_llm_b200.layers.losses import LanguageModelLossConfig, MonolithicLossConfig
    from fast_llm_b200.parallel.topology import DistributedConfig

    if type_name == "monolithic":  # built by the head from its combinable losses, never named in a config file
        config = MonolithicLossConfig.from_dict(fields)
    else:
        config = LanguageModelLossConfig.from_dict({"type": type_name, **(fields or {})})
    config.validate()
    distributed_config = DistributedConfig.from_dict({"world_size": 1, "rank": 0, "local_world_size": 1, "use_cuda": False})
    distributed_config.validate()
    layer = config.get_layer(distributed_config, name=type_name, vocab_parallel=group is not None)
    layer.setup(_Distributed(), group, vocab_begin)
    return layer


def _kwargs(labels, adv, old, doc, teacher=None, mask=None):
    from fast_llm_b200.layers.kwargs import LanguageModelKwargs as K

    kwargs = {K.labels: labels, K.advantages: adv, K.old_log_probabilities: old, K.document_index: doc}
    if teacher is not None:
        kwargs["teacher_logits"] = teacher
    if mask is not None:
        kwargs[K.loss_mask] = mask
    return kwargs


def _run_label_case(kind, scale, group=None, rank=0, world=1, device="cpu", dtype=torch.float32):
    logits, teacher, labels, adv, old, doc = _inputs()
    expected_value, expected_grad = _oracle_label(kind if kind != "label" else "cross_entropy", logits, labels, scale, adv, old, doc)
    shard = V // world
    local = logits[:, rank * shard : (rank + 1) * shard].contiguous().to(device=device, dtype=dtype)
    layer = _layer(kind, {"logits_scale_factor": 1.0}, group, rank * shard)
    kwargs = _kwargs(labels.to(device), adv.to(device), old.to(device), doc.to(device))
    value, grad = layer.forward_backward(local.clone(), kwargs, 1.0, 0, 1, scale)
    return value.float().cpu(), grad.float().cpu(), expected_value, expected_grad[:, rank * shard : (rank + 1) * shard]


@pytest.mark.parametrize("kind", ["label", "z_loss", "grpo", "gspo"])
@pytest.mark.parametrize("scale", [1.0, 0.5])
def test_label_based_losses_match_autograd(kind, scale):
    value, grad, expected_value, expected_grad = _run_label_case(kind, scale)
    torch.testing.assert_close(value, expected_value, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(grad, expected_grad, rtol=1e-4, atol=1e-7)


@pytest.mark.parametrize("kind", ["cross_entropy", "forward_kl", "reverse_kl"])
@pytest.mark.parametrize("masked", [False, True])
@pytest.mark.parametrize("temperature", [1.0, 2.0])
def test_distillation_losses_match_autograd(kind, masked, temperature):
    logits, teacher, labels, adv, old, doc = _inputs()
    mask = (labels >= 0).float() if masked else None
    expected_value, expected_grad = _oracle_distribution(kind, logits, teacher, mask, 1.0, temperature)
    layer = _layer("distillation", {"loss_type": kind, "temperature": temperature})
    value, grad = layer.forward_backward(logits.clone(), _kwargs(labels, adv, old, doc, teacher, mask), 1.0, 0, 1, 1.0)
    torch.testing.assert_close(value, expected_value, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(grad, expected_grad, rtol=1e-4, atol=1e-7)


def test_monolithic_loss_is_the_weighted_sum_in_one_gradient():
    logits, teacher, labels, adv, old, doc = _inputs()
    weights = {"label": 1.0, "z_loss": 1e-2, "grpo": 0.5}
    layer = _layer("monolithic", {"losses": {"ce": {"type": "label", "weight": weights["label"]}, "z": {"type": "z_loss", "weight": weights["z_loss"]},
                                             "pg": {"type": "grpo", "weight": weights["grpo"]}}})
    value, grad = layer.forward_backward(logits.clone(), _kwargs(labels, adv, old, doc), 1.0, 0, 1, 1.0)
    expected_value, expected_grad = 0.0, 0.0
    for kind, w in (("cross_entropy", weights["label"]), ("z_loss", weights["z_loss"]), ("grpo", weights["grpo"])):
        v, g = _oracle_label(kind, logits, labels, 1.0, adv, old, doc)
        expected_value, expected_grad = expected_value + w * v, expected_grad + w * g
    torch.testing.assert_close(value, expected_value, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(grad, expected_grad, rtol=1e-4, atol=1e-7)


def test_dpo_matches_autograd():
    logits, teacher, labels, adv, old, doc = _inputs(mask_some=False)
    chosen, rejected = [(2, 10), (20, 25)], [(10, 18), (30, 40)]
    from fast_llm_b200.layers.kwargs import LanguageModelKwargs as K

    kwargs = {K.labels: labels, K.chosen_spans: chosen, K.rejected_spans: rejected, "reference_logits": teacher}
    layer = _layer("dpo", {"beta": 0.7})
    value, grad = layer.forward_backward(logits.clone(), kwargs, 1.0, 0, 1, 1.0)
    x = logits.double().requires_grad_()
    lp = torch.log_softmax(x, -1).gather(-1, labels[:, None])[:, 0]
    ref = torch.log_softmax(teacher.double(), -1).gather(-1, labels[:, None])[:, 0]
    span = lambda v, spans: sum(v[b:e].sum() for b, e in spans)  # noqa: E731
    loss = -torch.nn.functional.logsigmoid(0.7 * ((span(lp, chosen) - span(lp, rejected)) - (span(ref, chosen) - span(ref, rejected))))
    (expected,) = torch.autograd.grad(loss, x)
    torch.testing.assert_close(value, loss.float(), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(grad, expected.float(), rtol=1e-4, atol=1e-7)


# ---------------------------------------------------------------------------------------------------------------------
# the reference's own PyTorch functions as a second oracle
@pytest.mark.skipif(not (REFERENCE / "fast_llm" / "functional" / "entropy_loss.py").exists(), reason="reference tree not present")
@pytest.mark.parametrize("loss_type", ["cross_entropy", "forward_kl", "reverse_kl"])
@pytest.mark.parametrize("target_format", ["labels", "logits"])
def test_entropy_losses_match_the_reference_functions(loss_type, target_format):
    old_flag = torch._dynamo.config.disable
    torch._dynamo.config.disable = True  # the reference decorates these functions with torch.compile
    sys.path.insert(0, str(REFERENCE))
    try:
        from fast_llm.functional.config import EntropyLossType, TargetFormat
        from fast_llm.functional.entropy_loss import torch_entropy_loss_forward_backward

        logits, teacher, labels, adv, old, doc = _inputs()
        if target_format == "labels":
            ref_value, ref_grad = torch_entropy_loss_forward_backward(logits, labels, None, 1.0, 1.0, TargetFormat.labels, EntropyLossType(loss_type))
            layer = _layer("label", {"loss_type": loss_type})
            value, grad = layer.forward_backward(logits.clone(), _kwargs(labels, adv, old, doc), 1.0, 0, 1, 1.0)
            # the reference function averages over all tokens, the layer over the labelled ones
            factor = (labels >= 0).sum() / T
            value, grad = value * factor, grad * factor
        else:
            mask = (labels >= 0).float()
            ref_value, ref_grad = torch_entropy_loss_forward_backward(logits, teacher, mask, 1.0, 1.0, TargetFormat.logits, EntropyLossType(loss_type),
                                                                      temperature=2.0)
            layer = _layer("distillation", {"loss_type": loss_type, "temperature": 2.0})
            value, grad = layer.forward_backward(logits.clone(), _kwargs(labels, adv, old, doc, teacher, mask), 1.0, 0, 1, 1.0)
            factor = mask.sum() / T
            value, grad = value * factor, grad * factor
        torch.testing.assert_close(value, ref_value, rtol=2e-5, atol=1e-6)
        torch.testing.assert_close(grad, ref_grad, rtol=2e-4, atol=1e-7)
    finally:
        torch._dynamo.config.disable = old_flag
        sys.path.remove(str(REFERENCE))
        for name in [n for n in sys.modules if n == "fast_llm" or n.startswith("fast_llm.")]:
            del sys.modules[name]


# ---------------------------------------------------------------------------------------------------------------------
# two vocabulary shards over Gloo
def _sharded_rank(rank, world, kind, extra):
    torch.distributed.init_process_group("gloo", rank=rank, world_size=world)
    group = torch.distributed.group.WORLD
    if kind == "distillation":
        logits, teacher, labels, adv, old, doc = _inputs()
        mask = (labels >= 0).float()
        expected_value, expected_grad = _oracle_distribution(extra, logits, teacher, mask, 1.0, 2.0)
        shard = V // world
        cols = slice(rank * shard, (rank + 1) * shard)
        layer = _layer("distillation", {"loss_type": extra, "temperature": 2.0}, group, rank * shard)
        value, grad = layer.forward_backward(logits[:, cols].contiguous(), _kwargs(labels, adv, old, doc, teacher[:, cols].contiguous(), mask), 1.0, 0, 1, 1.0)
        expected_grad = expected_grad[:, cols]
    else:
        value, grad, expected_value, expected_grad = _run_label_case(kind, 1.0, group, rank, world)
    torch.testing.assert_close(value, expected_value, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(grad, expected_grad, rtol=1e-4, atol=1e-7)
    return True


@pytest.mark.parametrize("kind,extra", [("label", None), ("z_loss", None), ("grpo", None), ("gspo", None), ("distillation", "cross_entropy"),
                                        ("distillation", "forward_kl"), ("distillation", "reverse_kl")])
def test_losses_over_two_vocabulary_shards(kind, extra):
    assert all(run_distributed(_sharded_rank, 2, kind, extra))


# ---------------------------------------------------------------------------------------------------------------------
# the CUDA kernels against the same oracles
@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["label", "z_loss", "grpo", "gspo"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_label_based_losses_gpu(kind, dtype):
    value, grad, expected_value, expected_grad = _run_label_case(kind, 0.5, device="cuda", dtype=dtype)
    tol = dict(rtol=1e-4, atol=1e-6) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-4)
    torch.testing.assert_close(value, expected_value, rtol=1e-4 if dtype == torch.float32 else 2e-2, atol=1e-5 if dtype == torch.float32 else 2e-2)
    torch.testing.assert_close(grad, expected_grad, **tol)


@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["cross_entropy", "forward_kl", "reverse_kl"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_distillation_losses_gpu(kind, dtype):
    logits, teacher, labels, adv, old, doc = _inputs()
    logits, teacher = logits.to(dtype).float(), teacher.to(dtype).float()  # the oracle sees the rounded inputs
    mask = (labels >= 0).float()
    expected_value, expected_grad = _oracle_distribution(kind, logits, teacher, mask, 1.0, 2.0)
    layer = _layer("distillation", {"loss_type": kind, "temperature": 2.0})
    kwargs = _kwargs(labels.cuda(), adv.cuda(), old.cuda(), doc.cuda(), teacher.cuda().to(dtype), mask.cuda())
    value, grad = layer.forward_backward(logits.cuda().to(dtype), kwargs, 1.0, 0, 1, 1.0)
    torch.testing.assert_close(value.float().cpu(), expected_value, rtol=1e-4, atol=1e-5)
    tol = dict(rtol=1e-4, atol=1e-7) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-5)
    torch.testing.assert_close(grad.float().cpu(), expected_grad, **tol)


@pytest.mark.gpu
def test_monolithic_loss_gpu_writes_one_gradient_in_place():
    from fast_llm_b200.ops import _lib

    logits, teacher, labels, adv, old, doc = _inputs()
    layer = _layer("monolithic", {"losses": {"ce": {"type": "label"}, "z": {"type": "z_loss", "weight": 1e-2}, "pg": {"type": "grpo", "weight": 0.5}}})
    device_logits = logits.cuda()
    before = _lib.launch_count
    value, grad = layer.forward_backward(device_logits, _kwargs(labels.cuda(), adv.cuda(), old.cuda(), doc.cuda()), 1.0, 0, 1, 1.0)
    assert _lib.launch_count - before == 2, "one statistics pass and one gradient pass for all three losses"
    assert grad.data_ptr() == device_logits.data_ptr()
    expected_value, expected_grad = 0.0, 0.0
    for kind, w in (("cross_entropy", 1.0), ("z_loss", 1e-2), ("grpo", 0.5)):
        v, g = _oracle_label(kind, logits, labels, 1.0, adv, old, doc)
        expected_value, expected_grad = expected_value + w * v, expected_grad + w * g
    torch.testing.assert_close(value.cpu(), expected_value, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(grad.cpu(), expected_grad, rtol=1e-4, atol=1e-7)


# ---------------------------------------------------------------------------------------------------------------------
# through the head: grouped (one softmax) and per-loss execution train identically
def test_head_groups_losses_sharing_the_softmax():
    from tests.common import build_trainer, tiny_trainer_config
    from fast_llm_b200.layers.losses import MonolithicLoss
    from fast_llm_b200.parallel.topology import PhaseType

    losses = {"lm_loss": {"type": "label"}, "z_loss": {"type": "z_loss", "weight": 1e-2}}
    results = {}
    for implementation in ("auto", "per_loss"):
        updates = {("model", "base_model", "head", "losses"): losses, ("model", "base_model", "head", "loss_implementation"): implementation,
                   ("model", "distributed", "reproducible_init"): True}
        trainer, _ = build_trainer(tiny_trainer_config(updates))
        head = trainer.multi_stage.base_model.head
        grouped = [type(l) for l in head._losses] == [MonolithicLoss]
        assert grouped == (implementation == "auto")
        schedule = trainer._schedules[PhaseType.training]
        iterator = trainer._data.get_iterator("training", consumed_samples=0, num_workers=0)
        out, ok, _ = trainer.runner.run_step(iterator, schedule, iteration=1)
        weights = {n: t.clone() for n, _, t in trainer.multi_stage.get_state_tensor_iterator(("weights",))}
        results[implementation] = (out, weights)
    auto, per_loss = results["auto"], results["per_loss"]
    assert set(auto[0]) >= {"lm_loss", "z_loss"}
    for name in ("lm_loss", "z_loss"):
        assert auto[0][name] == pytest.approx(per_loss[0][name], rel=1e-5)
    for name, value in auto[1].items():
        torch.testing.assert_close(value, per_loss[1][name], rtol=1e-3, atol=1e-4)  # Adam turns rounding differences of tiny gradients into steps of the order of the learning rate
