"""Generation-based evaluation (lm-evaluation-harness) and the stand-alone `fast-llm evaluate` command.

`FastLLMLmEvalWrapper` exposes the three requests of the harness' language-model interface - `loglikelihood`,
`loglikelihood_rolling`, `generate_until` - on top of the Hugging Face wrapper of a staged model.  It does not import
the harness itself, so it can be used (and is tested) without it; `LmEvalEvaluator` hands it to
`lm_eval.simple_evaluate` when the package is installed.  With tensor parallelism only the coordinator rank drives the
harness; the other ranks mirror its forward passes (`worker_forward`).
Parity: `fast_llm/engine/evaluation/lm_eval/evaluator.py`, `fast_llm_lm_eval_wrapper.py` (TemplateLM subclass, batching
by length, TP worker protocol), `fast_llm/engine/evaluation/config.py` (LmEvalEvaluatorConfig, `evaluate` runnable).
"""

import logging
import typing

import torch

from fast_llm_b200.config import Field, FieldHint, config_class
from fast_llm_b200.config.runnable import RunnableConfig
from fast_llm_b200.data.config import TokenizerConfig
from fast_llm_b200.engine.evaluation.evaluator import Evaluator
from fast_llm_b200.engine.training.config import EvaluatorConfig, TrainerConfig

logger = logging.getLogger(__name__)


@config_class(dynamic_type={EvaluatorConfig: "lm_eval"})
class LmEvalEvaluatorConfig(EvaluatorConfig):
    _abstract: typing.ClassVar[bool] = False
    tokenizer: TokenizerConfig = Field(desc="Tokenizer used to encode prompts and decode generations.", hint=FieldHint.core)
    tasks: list[str] = Field(default_factory=list, desc="Harness task names.", hint=FieldHint.core)
    num_fewshot: int | None = Field(default=None, desc="Few-shot examples per prompt.", hint=FieldHint.feature)
    limit: float | None = Field(default=None, desc="Documents per task (count, or fraction below 1).", hint=FieldHint.feature)
    batch_size: int = Field(default=8, desc="Sequences scored per forward pass.", hint=FieldHint.performance)
    max_length: int | None = Field(default=None, desc="Context limit (longer prompts are left-truncated).", hint=FieldHint.feature)
    max_new_tokens: int = Field(default=256, desc="Default generation budget.", hint=FieldHint.feature)
    add_bos_token: bool = Field(default=False, desc="Prepend the beginning-of-document token to contexts.", hint=FieldHint.feature)
    cli_args: list[str] = Field(default_factory=list, desc="Extra arguments for `simple_evaluate`: `key=value` items or the harness' own command line (`--tasks a,b --num_fewshot 5 ...`).", hint=FieldHint.optional)

    def get_evaluator(self, name, *args, **kwargs):
        return LmEvalEvaluator(name, self)


class FastLLMLmEvalWrapper:
    """Scores and generates with a `HuggingfacePreTrainedModel`.  Requests are the harness' `Instance`s or plain tuples
    (anything with `.args`, or the argument tuple itself)."""

    def __init__(self, model, tokenizer, *, batch_size: int = 8, max_length: int | None = None, max_new_tokens: int = 256,
                 add_bos_token: bool = False, data_group=None):
        """`data_group`: the process group of the model replicas (batch-data parallel).  Every replica's coordinator runs the same
        harness code on the same requests; with a group each scores / generates every n-th request and the results are
        exchanged, so the replicas share the work instead of repeating it."""
        self._model, self._tokenizer = model, tokenizer
        self._data_group = data_group if (data_group is not None and data_group.size() > 1) else None
        self.batch_size, self._max_length = batch_size, max_length or 2**30
        self._max_new_tokens, self._add_bos = max_new_tokens, add_bos_token
        self.device = model.fast_llm_model.distributed.device

    # ---- helpers
    @property
    def eot_token_id(self) -> int:
        return self._tokenizer.eod_id

    @property
    def tokenizer_name(self) -> str:
        return str(self._tokenizer._config.path)

    @property
    def prefix_token_id(self) -> int:
        """The token that stands in for an empty context (the harness scores `P(continuation | prefix)`)."""
        return self._tokenizer.bod_id if self._tokenizer.bod_id is not None else self.eot_token_id

    @property
    def max_length(self) -> int:
        return self._max_length

    @property
    def max_gen_toks(self) -> int:
        return self._max_new_tokens

    # the harness runs in one process per model replica here: it sees one rank
    rank, world_size = 0, 1

    def apply_chat_template(self, chat_history: list[dict[str, str]], add_generation_prompt: bool = True) -> str:
        """Render a list of {"role", "content"} messages with the tokenizer's chat template (needed for `--apply_chat_template`)."""
        inner = getattr(self._tokenizer, "tokenizer", None)
        if inner is not None and getattr(inner, "chat_template", None):
            return inner.apply_chat_template(chat_history, tokenize=False, add_generation_prompt=add_generation_prompt)
        text = "".join(f"{m['role']}: {m['content']}\n" for m in chat_history)  # plain fallback for tokenizers without a template
        return text + ("assistant: " if add_generation_prompt else "")

    def tok_batch_encode(self, texts: list[str], left_truncate_len: int | None = None) -> tuple[torch.Tensor, torch.Tensor]:
        """Left-padded token batch and its attention mask."""
        rows = [self.tok_encode(t) for t in texts]
        if left_truncate_len is not None:
            rows = [r[-left_truncate_len:] for r in rows]
        width = max((len(r) for r in rows), default=0)
        pad = self.eot_token_id or 0
        ids = torch.tensor([[pad] * (width - len(r)) + r for r in rows], dtype=torch.int64, device=self.device)
        mask = torch.tensor([[0] * (width - len(r)) + [1] * len(r) for r in rows], dtype=torch.int64, device=self.device)
        return ids, mask

    @staticmethod
    def _args(request):
        return request.args if hasattr(request, "args") else request

    def tok_encode(self, text: str) -> list[int]:
        return self._tokenizer.tokenize(text, begin=False, end=False).tolist()

    def tok_decode(self, tokens) -> str:
        return self._tokenizer.detokenize(list(tokens))

    def _encode_pair(self, context: str, continuation: str) -> tuple[list[int], list[int]]:
        """Trailing spaces of the context belong to the continuation (they tokenize with the following word)."""
        stripped = context.rstrip()
        continuation = context[len(stripped):] + continuation
        whole = self.tok_encode(stripped + continuation)
        context_tokens = self.tok_encode(stripped)
        if not context_tokens:
            context_tokens = [self._tokenizer.bod_id if self._tokenizer.bod_id is not None else self.eot_token_id]
            return context_tokens, whole
        return context_tokens, whole[len(context_tokens):]

    def _shared(self, items: list, compute) -> list:
        """`compute(items)` with the items dealt out over the model replicas (round robin) and the results put back in order."""
        if self._data_group is None:
            return compute(items)
        rank, size = self._data_group.rank(), self._data_group.size()
        mine = list(range(rank, len(items), size))
        local = compute([items[i] for i in mine]) if mine else []
        gathered: list = [None] * size
        torch.distributed.all_gather_object(gathered, (mine, local), group=self._data_group)
        out: list = [None] * len(items)
        for indices, values in gathered:
            for index, value in zip(indices, values):
                out[index] = value
        return out

    def _score(self, sequences: list[tuple[list[int], list[int]]]) -> list[tuple[float, bool]]:
        return self._shared(sequences, self._score_local)

    def _score_local(self, sequences: list[tuple[list[int], list[int]]]) -> list[tuple[float, bool]]:
        """For each (context, continuation): sum of continuation log-probabilities, and whether it is the greedy choice."""
        results: list[tuple[float, bool] | None] = [None] * len(sequences)
        order = sorted(range(len(sequences)), key=lambda i: -(len(sequences[i][0]) + len(sequences[i][1])))
        for start in range(0, len(order), self.batch_size):
            chunk = order[start : start + self.batch_size]
            rows = []
            for i in chunk:
                context, continuation = sequences[i]
                tokens = (context + continuation)[-(self._max_length + 1):][:-1]  # inputs: everything but the last target
                rows.append(tokens)
            width = max(len(r) for r in rows)
            pad = self.eot_token_id or 0
            input_ids = torch.tensor([[pad] * (width - len(r)) + r for r in rows], dtype=torch.int64, device=self.device)
            mask = torch.tensor([[0] * (width - len(r)) + [1] * len(r) for r in rows], dtype=torch.int64, device=self.device)
            logits = self._model(input_ids=input_ids, attention_mask=mask).logits.float()
            log_probs = torch.log_softmax(logits, dim=-1)
            for row, i in enumerate(chunk):
                continuation = sequences[i][1]
                n = len(continuation)
                targets = torch.tensor(continuation, dtype=torch.int64, device=self.device)
                rows_lp = log_probs[row, width - n :]
                total = rows_lp.gather(1, targets[:, None]).sum().item()
                greedy = bool((rows_lp.argmax(-1) == targets).all())
                results[i] = (total, greedy)
        return results

    # ---- the three request types
    def loglikelihood(self, requests) -> list[tuple[float, bool]]:
        pairs = []
        for request in requests:
            context, continuation = self._args(request)[:2]
            context_tokens, continuation_tokens = self._encode_pair(context, continuation)
            if self._add_bos and self._tokenizer.bod_id is not None:
                context_tokens = [self._tokenizer.bod_id, *context_tokens]
            pairs.append((context_tokens, continuation_tokens))
        return self._score(pairs)

    def loglikelihood_rolling(self, requests) -> list[float]:
        return self._shared(list(requests), self._rolling_local)

    def _rolling_local(self, requests) -> list[float]:
        """Log-likelihood of whole documents, in windows of the context limit (each token scored once)."""
        out = []
        for request in requests:
            (text,) = self._args(request)[:1]
            tokens = self.tok_encode(text)
            prefix = [self._tokenizer.bod_id if self._tokenizer.bod_id is not None else self.eot_token_id]
            total, position = 0.0, 0
            window = min(self._max_length, 2**20)
            while position < len(tokens):
                targets = tokens[position : position + window]
                context = prefix if position == 0 else tokens[max(position - 1, 0) : position]
                total += self._score_local([(context, targets)])[0][0]
                position += len(targets)
            out.append(total)
        return out

    def generate_until(self, requests) -> list[str]:
        return self._shared(list(requests), self._generate_local)

    def _generate_local(self, requests) -> list[str]:
        """Requests are grouped by their generation options and sorted by prompt length, then generated `batch_size` at a time
        (left-padded); every answer is cut at the first of its stop strings."""
        prepared = []
        for index, request in enumerate(requests):
            context, options = self._args(request)[:2]
            options = dict(options or {})
            until = options.pop("until", None) or []
            until = [until] if isinstance(until, str) else list(until)
            budget = int(options.pop("max_gen_toks", self._max_new_tokens))
            tokens = self.tok_encode(context)
            if self._add_bos and self._tokenizer.bod_id is not None:
                tokens = [self._tokenizer.bod_id, *tokens]
            tokens = tokens[-max(self._max_length - budget, 1):]
            key = (budget, bool(options.get("do_sample", False)), float(options.get("temperature", 0.0) or 0.0), tuple(until))
            prepared.append((key, len(tokens), index, tokens))
        out: list[str | None] = [None] * len(prepared)
        prepared.sort(key=lambda item: (item[0], -item[1]))
        start = 0
        while start < len(prepared):
            key = prepared[start][0]
            chunk = [item for item in prepared[start : start + self.batch_size] if item[0] == key]
            start += len(chunk)
            budget, do_sample, temperature, until = key
            width = max(item[1] for item in chunk)
            pad = self.eot_token_id or 0
            input_ids = torch.tensor([[pad] * (width - n) + tokens for _, n, _, tokens in chunk], dtype=torch.int64, device=self.device)
            mask = torch.tensor([[0] * (width - n) + [1] * n for _, n, _, _ in chunk], dtype=torch.int64, device=self.device)
            sampling = {"do_sample": True, "temperature": temperature} if (do_sample and temperature > 0) else {"do_sample": False}
            generated = self._model.generate(input_ids, attention_mask=mask, max_new_tokens=budget, pad_token_id=pad,
                                             eos_token_id=self.eot_token_id, **sampling)
            for row, (_, _, index, _) in enumerate(chunk):
                new_tokens = generated[row, width:].tolist()
                if self.eot_token_id in new_tokens:
                    new_tokens = new_tokens[: new_tokens.index(self.eot_token_id)]
                text = self.tok_decode(new_tokens)
                for stop in until:
                    if stop and stop in text:
                        text = text.split(stop)[0]
                out[index] = text
        return out


def parse_harness_arguments(cli_args: list[str]) -> dict:
    """Arguments for `lm_eval.simple_evaluate` from either spelling: `key=value` items, or the harness' own command line
    (`--tasks a,b --num_fewshot 5 --limit 0.1 --apply_chat_template --gen_kwargs temperature=0,top_p=1`).  Numbers, booleans
    and `None` are converted; `tasks` becomes a list."""
    def convert(value: str):
        lowered = value.lower()
        if lowered in ("true", "false"):
            return lowered == "true"
        if lowered in ("none", "null"):
            return None
        for kind in (int, float):
            try:
                return kind(value)
            except ValueError:
                pass
        return value

    out: dict = {}
    index = 0
    while index < len(cli_args):
        item = cli_args[index]
        if item.startswith("--"):
            key = item[2:].replace("-", "_")
            if "=" in key:
                key, value = key.split("=", 1)
                out[key] = convert(value)
            elif index + 1 < len(cli_args) and not cli_args[index + 1].startswith("--"):
                index += 1
                out[key] = convert(cli_args[index])
            else:
                out[key] = True  # a flag
        elif "=" in item:
            key, value = item.split("=", 1)
            out[key] = convert(value)
        else:
            raise ValueError(f"cannot parse harness argument {item!r}")
        index += 1
    if isinstance(out.get("tasks"), str):
        out["tasks"] = [t for t in out["tasks"].split(",") if t]
    if isinstance(out.get("gen_kwargs"), str):
        out["gen_kwargs"] = {k: convert(v) for k, v in (pair.split("=", 1) for pair in out["gen_kwargs"].split(","))}
    return out


class LmEvalEvaluator(Evaluator):
    def setup(self, trainer, distributed, run) -> None:
        super().setup(trainer, distributed, run)
        from fast_llm_b200.engine.inference.huggingface import HuggingfaceGPTModelForCausalLM

        self._hf_model = HuggingfaceGPTModelForCausalLM(trainer.multi_stage)
        self._wrapper = FastLLMLmEvalWrapper(self._hf_model, self._config.tokenizer.get_tokenizer(), batch_size=self._config.batch_size,
                                             max_length=self._config.max_length, max_new_tokens=self._config.max_new_tokens,
                                             add_bos_token=self._config.add_bos_token, data_group=getattr(distributed, "batch_data_group", None))

    def run(self, completed_steps: int, force: bool = False) -> dict | None:
        if not (force or self._config.enabled(completed_steps)):
            return None
        is_coordinator = self._distributed.config.tensor_rank == 0
        if not is_coordinator:
            self._hf_model.worker_forward()
            return None
        try:
            import lm_eval
        except ImportError as e:
            self._hf_model.stop_workers()
            raise ImportError("The lm_eval evaluator needs the `lm_eval` package (lm-evaluation-harness)") from e
        arguments = {"tasks": list(self._config.tasks), "num_fewshot": self._config.num_fewshot, "limit": self._config.limit,
                     **parse_harness_arguments(self._config.cli_args)}
        try:
            results = lm_eval.simple_evaluate(model=_as_harness_model(self._wrapper), **arguments)
        finally:
            self._hf_model.stop_workers()
        metrics = {task: {k: v for k, v in values.items() if isinstance(v, (int, float))} for task, values in results["results"].items()}
        try:  # the harness' own table, as its command line prints it
            from lm_eval.utils import make_table

            logger.info(f"lm_eval [{self._name}] step {completed_steps}:\n{make_table(results)}")
        except Exception:
            logger.info(f"lm_eval [{self._name}] step {completed_steps}: {metrics}")
        return {f"lm_eval.{self._name}": metrics}


def _as_harness_model(wrapper: FastLLMLmEvalWrapper):
    """Subclass the harness' `LM` at run time so the wrapper module itself never imports the harness."""
    from lm_eval.api.model import LM

    class _Model(LM):
        def loglikelihood(self, requests):
            return wrapper.loglikelihood(requests)

        def loglikelihood_rolling(self, requests):
            return wrapper.loglikelihood_rolling(requests)

        def generate_until(self, requests):
            return wrapper.generate_until(requests)

        def apply_chat_template(self, chat_history, add_generation_prompt=True):
            return wrapper.apply_chat_template(chat_history, add_generation_prompt)

        @property
        def tokenizer_name(self):
            return wrapper.tokenizer_name

        @property
        def eot_token_id(self):
            return wrapper.eot_token_id

        @property
        def max_length(self):
            return wrapper.max_length

    return _Model()


@config_class(dynamic_type={RunnableConfig: "evaluate"})
class EvaluatorsRunnableConfig(RunnableConfig):
    """`fast-llm evaluate <trainer type> -c config.yaml`: load the pretrained model of a training config and run its evaluators once."""

    _abstract: typing.ClassVar[bool] = True

    @classmethod
    def parse_and_run(cls, args: list[str] | None = None):
        import sys

        args = list(sys.argv[1:] if args is None else args)
        trainer_class = TrainerConfig.get_subclass(args[0]) if args and not args[0].startswith("-") and "=" not in args[0] else TrainerConfig
        remaining = args[1:] if trainer_class is not TrainerConfig else args
        parser = trainer_class._get_parser()
        parsed, unparsed = parser.parse_known_args(remaining)
        from fast_llm_b200.config import NoAutoValidate

        with NoAutoValidate():
            config = trainer_class._from_parsed_args(parsed, [*unparsed, "training.train_iters=0"])
        config.configure_logging()
        config.validate()
        if not parsed.do_run:
            return config
        return config._get_runnable()()
