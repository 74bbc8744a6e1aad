"""One-line formatting of training / validation metrics (parity: `fast_llm/logging.py:36-124`)."""

import datetime


def _fmt_time(seconds: float) -> str:
    return str(datetime.timedelta(seconds=int(max(seconds, 0))))


def format_metrics(metrics: dict, loss_defs, phase, dataset_name: str | None = None) -> str:
    name = getattr(phase, "value", str(phase)) + (f" @ {dataset_name}" if dataset_name else "")
    parts = [f"{name} iteration {metrics.get('iteration', 0):>6}/{metrics.get('train_iters', 0)}"]
    if "consumed_samples" in metrics:
        parts.append(f"consumed samples: {metrics['consumed_samples']:>9,}")
        parts.append(f"consumed tokens: {metrics['consumed_tokens']:>13,}")
    if "step_time_ms" in metrics:
        parts.append(f"step time {metrics['step_time_ms']:.2f} ms")
    if "tokens_per_sec_per_gpu" in metrics:
        parts.append(f"throughput {metrics.get('model_tflops', float('nan')):.2f} tflop/s (model) | "
                     f"{metrics.get('hardware_tflops', float('nan')):.2f} tflop/s (hardware) | "
                     f"{metrics['tokens_per_sec_per_gpu']:.2f} tokens/s/gpu")
    if "allocated" in metrics:
        parts.append(f"Memory allocated {metrics['allocated']:,.2f} MiB | max allocated {metrics['max_allocated']:,.2f} MiB | "
                     f"reserved {metrics['reserved']:,.2f} MiB | max reserved {metrics['max_reserved']:,.2f} MiB")
    if "learning_rate" in metrics:
        parts.append(f"learning rate {metrics['learning_rate']:.3e}")
    if "loss_scale" in metrics:
        parts.append(f"loss scale {metrics['loss_scale']:>8.0f}")
    if "grad_norm" in metrics:
        parts.append(f"grad norm {metrics['grad_norm']:.4f}")
    if "skipped_iters" in metrics:
        parts.append(f"skipped iterations {metrics['skipped_iters']:>3} | nan iterations {metrics['nan_iters']:>3}")
    if "data_wait_ms" in metrics:
        parts.append(f"data wait {metrics['data_wait_ms']:.1f} ms | preprocess {metrics.get('preprocess_ms', 0):.1f} ms")
    if "step_time_average_ms" in metrics:
        parts.append(f"average step time {metrics['step_time_average_ms']:.2f} ms | remaining {_fmt_time(metrics.get('remaining_time', 0))}"
                     f" | completion {datetime.datetime.fromtimestamp(metrics.get('completion_time', 0)).strftime('%Y-%m-%d %H:%M:%S')}"
                     f" ({metrics.get('percent_done', 0):.2f} %)")
    for loss_def in loss_defs:
        if loss_def.name in metrics:
            parts.append(f"{loss_def.formatted_name}: {metrics[loss_def.name]:.5f}")
    return " | ".join(parts)
