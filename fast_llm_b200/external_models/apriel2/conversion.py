"""Surgery on Apriel2 checkpoints: change the mixers of a model and carry the weights over.

Three layers, each usable alone (same roles as `fast_llm_external_models/apriel2/conversion/{config,expr,converters,executor}.py`,
own design):

**Configuration algebra.**  A *state* is a complete Apriel2 text configuration (a dict).  A *surgery* is a partial configuration
that names what changes; it may carry `init: transfer | random` next to a component to say where that component's weights come
from.  `compose_configs(state, surgery)` gives the *transition*: the complete target configuration with the `init` marks still
in it; `strip_init_fields` turns a transition into the state that is written to disk.  Surgeries also compose with each other
(`compose_configs(surgery, surgery)` is a deep merge), and for surgeries that do not replace a component's type applying them
one after the other equals applying their merge.  When a surgery changes a mixer's `type`, what the new type can inherit from
the old one is derived (attention heads -> delta-net value heads, and so on); wrapping a mixer into a `stochastic` mixer keeps
the old mixer as the sub-mixer that declares no type of its own.

**Plans.**  A plan maps every tensor of the target checkpoint to an expression over the tensors of the source checkpoint:
`Ref` (take a tensor), `Slice`, `Concat`, `Reshape` and `Init` (new values: normal, zeros, ones, or the log of a uniform range
for decay rates).  Plans are data: they print, serialise (`to_dict` / `from_dict`), and compose by substitution
(`compose_plans(first, then)`), so a chain of surgeries runs as one pass over the source tensors.  Random values depend only on
the seed and on the name recorded in the `Init` node, not on evaluation order.

**Planning.**  `plan_surgery(source_state, transition)` builds the plan: unchanged components are references; an attention
mixer turned into a Mamba mixer is initialised from it (x <- value, B <- key, C <- query projection rows, output projection kept:
the "Mamba in the Llama" initialisation), into a gated delta-net or Kimi delta attention likewise (key / value rows repeated
over the heads of a group where the target has no grouped heads); everything else of a new component is `Init`.  Target tensor
names and shapes come from building the target model on the meta device, so the plan cannot drift from the modelling code.

Command line: `python -m fast_llm_b200.external_models.apriel2.conversion <input dir> <output dir> --surgery a.yaml [--surgery b.yaml ...]`.
"""

import argparse
import copy
import hashlib
import json
import math
import pathlib
import typing

import torch

INIT_KEY = "init"

# ---------------------------------------------------------------------------------------------- configuration algebra


def _is_mixer(node: dict) -> bool:
    return isinstance(node, dict) and ("heads" in node or "mixers" in node or node.get("type") in _MIXER_TYPES)


_MIXER_TYPES = ("attention", "mamba", "gdn", "kda", "stochastic")


def _derive_mixer(base: dict, new_type: str, hidden_size: int | None) -> dict:
    """What a mixer of `new_type` inherits from the mixer it replaces."""
    base_type = base.get("type", "attention")
    if base_type == "stochastic":
        main = base.get("main_mixer_name") or next(iter(base["mixers"]))
        return _derive_mixer(base["mixers"][main], new_type, hidden_size)
    if base_type == new_type:
        return copy.deepcopy(base)
    if base_type != "attention":
        return {}
    heads, groups, size = base["heads"], base.get("head_groups", base["heads"]), base["head_size"]
    if new_type == "gdn":
        return {"value_heads": heads, "key_heads": groups, "key_head_dim": size, "value_head_dim": size}
    if new_type == "kda":
        return {"heads": heads, "head_dim": size}
    if new_type == "mamba":
        out = {"d_inner": heads * size, "d_xb": groups * size, "state_size": 16, "add_linear_biases": False}
        if hidden_size is not None:
            out["dt_rank"] = math.ceil(hidden_size / 16)
        return out
    return {}


def _merge(base, patch, hidden_size=None):
    """Deep merge with the mixer rules of the module docstring."""
    if not isinstance(base, dict) or not isinstance(patch, dict):
        return copy.deepcopy(patch)
    if _is_mixer(base) and "type" in patch and patch["type"] != base.get("type", "attention"):
        new_type = patch["type"]
        if new_type == "stochastic":
            mixers = {}
            for name, sub in patch.get("mixers", {}).items():
                if "type" in sub and sub["type"] != base.get("type", "attention"):
                    mixers[name] = _merge(base, sub, hidden_size)
                else:  # the sub-mixer that declares no other type is the mixer that was there
                    mixers[name] = _merge(base, {INIT_KEY: "transfer", **sub}, hidden_size)
            out = {k: copy.deepcopy(v) for k, v in patch.items() if k != "mixers"}
            out["mixers"] = mixers
            out.setdefault("main_mixer_name", next(iter(mixers)))
            return out
        derived = _derive_mixer(base, new_type, hidden_size)
        out = {**derived, **{k: copy.deepcopy(v) for k, v in patch.items()}}
        out.setdefault(INIT_KEY, "transfer")
        return out
    out = copy.deepcopy(base)
    for key, value in patch.items():
        if key == "mixers" and isinstance(value, dict) and isinstance(out.get("mixers"), dict):
            main = out.get("main_mixer_name") or next(iter(out["mixers"]))
            for name, sub in value.items():
                if name in out["mixers"]:
                    out["mixers"][name] = _merge(out["mixers"][name], sub, hidden_size)
                else:  # a new sub-mixer is described relative to the main one
                    out["mixers"][name] = _merge(out["mixers"][main], sub, hidden_size)
        elif key in out and isinstance(out[key], dict) and isinstance(value, dict):
            out[key] = _merge(out[key], value, hidden_size)
        else:
            out[key] = copy.deepcopy(value)
    return out


def compose_configs(base: dict, surgery: dict) -> dict:
    """state x surgery -> transition; transition x surgery -> transition; surgery x surgery -> surgery."""
    hidden_size = surgery.get("hidden_size", base.get("hidden_size"))
    out = {k: copy.deepcopy(v) for k, v in base.items() if k != "decoder"}
    for key, value in surgery.items():
        if key != "decoder":
            out[key] = _merge(out.get(key), value, hidden_size) if key in out else copy.deepcopy(value)
    base_decoder, patch_decoder = base.get("decoder"), surgery.get("decoder")
    if patch_decoder is None:
        if base_decoder is not None:
            out["decoder"] = copy.deepcopy(base_decoder)
        return out
    if base_decoder is None:
        out["decoder"] = copy.deepcopy(patch_decoder)
        return out
    base_kind, patch_kind = base_decoder.get("type", "fixed"), patch_decoder.get("type", base_decoder.get("type", "fixed"))
    if base_kind == "fixed" and patch_kind == "pattern":
        # every named block of the pattern is described relative to the one block of the fixed decoder
        blocks = {name: _merge(base_decoder["block"], block, hidden_size) for name, block in patch_decoder.get("blocks", {}).items()}
        decoder = {"type": "pattern", "num_blocks": patch_decoder.get("num_blocks", base_decoder["num_blocks"]),
                   "pattern": list(patch_decoder["pattern"]), "blocks": blocks}
    elif base_kind == "pattern" and patch_kind == "pattern":
        decoder = copy.deepcopy(base_decoder)
        for key, value in patch_decoder.items():
            if key == "blocks":
                for name, block in value.items():
                    relative_to = decoder["blocks"].get(name) or next(iter(decoder["blocks"].values()))
                    decoder["blocks"][name] = _merge(relative_to, block, hidden_size)
            else:
                decoder[key] = copy.deepcopy(value)
    else:
        decoder = _merge(base_decoder, patch_decoder, hidden_size)
    out["decoder"] = decoder
    return out


def strip_init_fields(config):
    """transition -> state: the same configuration without the `init` marks."""
    if isinstance(config, dict):
        return {k: strip_init_fields(v) for k, v in config.items() if k != INIT_KEY}
    if isinstance(config, list):
        return [strip_init_fields(v) for v in config]
    return config


def block_configs(state: dict) -> list[dict]:
    decoder = state["decoder"]
    if decoder.get("type", "fixed") == "fixed":
        return [decoder["block"]] * decoder["num_blocks"]
    pattern = decoder["pattern"]
    return [decoder["blocks"][pattern[i % len(pattern)]] for i in range(decoder["num_blocks"])]


# ---------------------------------------------------------------------------------------------- expressions and plans


class Expr:
    def evaluate(self, source: typing.Mapping[str, torch.Tensor], seed: int) -> torch.Tensor:
        raise NotImplementedError

    def substitute(self, plan: "Plan") -> "Expr":
        """The same expression over the sources of `plan` (every reference replaced by what `plan` builds for that name)."""
        raise NotImplementedError

    def references(self) -> set[str]:
        raise NotImplementedError

    def to_dict(self) -> dict:
        raise NotImplementedError

    @staticmethod
    def from_dict(data: dict) -> "Expr":
        kind = data["op"]
        if kind == "ref":
            return Ref(data["key"])
        if kind == "slice":
            return Slice(Expr.from_dict(data["of"]), data["dim"], data["start"], data["stop"])
        if kind == "concat":
            return Concat([Expr.from_dict(e) for e in data["of"]], data["dim"])
        if kind == "reshape":
            return Reshape(Expr.from_dict(data["of"]), tuple(data["shape"]))
        if kind == "init":
            return Init(tuple(data["shape"]), data["kind"], data["name"], data.get("scale", 0.02), data.get("dtype", "float32"))
        raise ValueError(f"unknown expression {kind!r}")


class Ref(Expr):
    def __init__(self, key: str):
        self.key = key

    def evaluate(self, source, seed):
        return source[self.key]

    def substitute(self, plan):
        return plan[self.key]

    def references(self):
        return {self.key}

    def to_dict(self):
        return {"op": "ref", "key": self.key}

    def __repr__(self):
        return f"Ref({self.key})"


class Slice(Expr):
    def __init__(self, of: Expr, dim: int, start: int, stop: int):
        self.of, self.dim, self.start, self.stop = of, dim, start, stop

    def evaluate(self, source, seed):
        return self.of.evaluate(source, seed).narrow(self.dim, self.start, self.stop - self.start)

    def substitute(self, plan):
        return Slice(self.of.substitute(plan), self.dim, self.start, self.stop)

    def references(self):
        return self.of.references()

    def to_dict(self):
        return {"op": "slice", "of": self.of.to_dict(), "dim": self.dim, "start": self.start, "stop": self.stop}

    def __repr__(self):
        return f"{self.of!r}[dim {self.dim}: {self.start}:{self.stop}]"


class Concat(Expr):
    def __init__(self, of: list[Expr], dim: int):
        self.of, self.dim = list(of), dim

    def evaluate(self, source, seed):
        parts = [e.evaluate(source, seed) for e in self.of]
        dtype = parts[0].dtype
        return torch.cat([p.to(dtype) for p in parts], dim=self.dim)

    def substitute(self, plan):
        return Concat([e.substitute(plan) for e in self.of], self.dim)

    def references(self):
        return set().union(*(e.references() for e in self.of)) if self.of else set()

    def to_dict(self):
        return {"op": "concat", "of": [e.to_dict() for e in self.of], "dim": self.dim}

    def __repr__(self):
        return f"Concat(dim {self.dim}: {', '.join(map(repr, self.of))})"


class Reshape(Expr):
    def __init__(self, of: Expr, shape: tuple[int, ...]):
        self.of, self.shape = of, tuple(shape)

    def evaluate(self, source, seed):
        return self.of.evaluate(source, seed).reshape(self.shape)

    def substitute(self, plan):
        return Reshape(self.of.substitute(plan), self.shape)

    def references(self):
        return self.of.references()

    def to_dict(self):
        return {"op": "reshape", "of": self.of.to_dict(), "shape": list(self.shape)}

    def __repr__(self):
        return f"Reshape({self.of!r}, {self.shape})"


class Init(Expr):
    """New values.  `kind`: normal (std `scale`), zeros, ones, log_uniform (log of uniform [1, 16]: decay rates).  The values
    depend on (seed, name) only."""

    def __init__(self, shape: tuple[int, ...], kind: str, name: str, scale: float = 0.02, dtype: str = "float32"):
        self.shape, self.kind, self.name, self.scale, self.dtype = tuple(shape), kind, name, scale, dtype

    def evaluate(self, source, seed):
        dtype = getattr(torch, self.dtype)
        if self.kind == "zeros":
            return torch.zeros(self.shape, dtype=dtype)
        if self.kind == "ones":
            return torch.ones(self.shape, dtype=dtype)
        digest = hashlib.sha256(f"{seed}:{self.name}".encode()).digest()
        generator = torch.Generator().manual_seed(int.from_bytes(digest[:8], "little") >> 1)
        if self.kind == "normal":
            return (torch.randn(self.shape, generator=generator) * self.scale).to(dtype)
        if self.kind == "log_uniform":
            return torch.log(1 + 15 * torch.rand(self.shape, generator=generator)).to(dtype)
        raise ValueError(self.kind)

    def substitute(self, plan):
        return self

    def references(self):
        return set()

    def to_dict(self):
        return {"op": "init", "shape": list(self.shape), "kind": self.kind, "name": self.name, "scale": self.scale, "dtype": self.dtype}

    def __repr__(self):
        return f"Init({self.kind}, {self.shape})"


class Plan(dict):
    """target tensor name -> expression over source tensor names."""

    def execute(self, source: typing.Mapping[str, torch.Tensor], seed: int = 0) -> dict[str, torch.Tensor]:
        return {name: expr.evaluate(source, seed).clone() for name, expr in self.items()}

    def stream(self, source: typing.Mapping[str, torch.Tensor], seed: int = 0) -> typing.Iterator[tuple[str, torch.Tensor]]:
        """One target tensor at a time (the source mapping may load lazily)."""
        for name, expr in self.items():
            yield name, expr.evaluate(source, seed).contiguous()

    def source_keys(self) -> set[str]:
        return set().union(*(e.references() for e in self.values())) if self else set()

    def to_dict(self) -> dict:
        return {name: expr.to_dict() for name, expr in self.items()}

    @classmethod
    def from_dict(cls, data: dict) -> "Plan":
        return cls({name: Expr.from_dict(expr) for name, expr in data.items()})

    def summary(self) -> str:
        kinds = {"kept": 0, "built": 0, "new": 0}
        for expr in self.values():
            kinds["kept" if isinstance(expr, Ref) else ("new" if isinstance(expr, Init) else "built")] += 1
        return f"{len(self)} tensors: {kinds['kept']} kept, {kinds['built']} built from source tensors, {kinds['new']} newly initialised"


def compose_plans(first: Plan, then: Plan) -> Plan:
    """The plan that gives what `then` gives when it is fed the output of `first`."""
    return Plan({name: expr.substitute(first) for name, expr in then.items()})


# ---------------------------------------------------------------------------------------------- planning


def _shapes(state: dict) -> dict[str, tuple[tuple[int, ...], str]]:
    """name -> (shape, dtype) of every parameter of the model this state describes (built on the meta device)."""
    try:
        from fast_llm_b200.external_models.apriel2.configuration_apriel2 import Apriel2TextConfig
        from fast_llm_b200.external_models.apriel2.modeling_apriel2 import Apriel2ForCausalLM
    except ImportError:  # pragma: no cover - next to an exported checkpoint
        from configuration_apriel2 import Apriel2TextConfig
        from modeling_apriel2 import Apriel2ForCausalLM

    fields = {k: v for k, v in state.items() if k not in ("model_type", "architectures", "auto_map", "torch_dtype", "dtype", "transformers_version")}
    with torch.device("meta"):
        model = Apriel2ForCausalLM(Apriel2TextConfig(**fields))
    out = {name: (tuple(p.shape), str(p.dtype).removeprefix("torch.")) for name, p in model.named_parameters()}
    if state.get("tie_word_embeddings", False):
        out.pop("lm_head.weight", None)
    return out


def _new_values(name: str, shape: tuple[int, ...], scale: float) -> Init:
    leaf = name.rsplit(".", 2)[-2:] if name.count(".") else [name]
    last = name.rsplit(".", 1)[-1]
    if last == "bias":
        kind = "zeros"
    elif last == "A_log":
        kind = "log_uniform"
    elif last in ("D", "dt_bias") or (last == "weight" and ("norm" in leaf[0])):
        kind = "ones"
    else:
        kind = "normal"
    return Init(shape, kind, name, scale)


def _rows(expr: Expr, start: int, stop: int) -> Expr:
    return Slice(expr, 0, start, stop)


def _repeat_groups(expr: Expr, groups: int, heads: int, size: int) -> Expr:
    """Rows of `groups` heads of `size` repeated so that every one of `heads` heads has the rows of its group."""
    if groups == heads:
        return expr
    ratio = heads // groups
    return Concat([_rows(expr, (h // ratio) * size, (h // ratio + 1) * size) for h in range(heads)], 0)


def _first_of_groups(expr: Expr, groups: int, heads: int, size: int) -> Expr:
    """Rows of the first head of every group."""
    if groups == heads:
        return expr
    ratio = heads // groups
    return Concat([_rows(expr, g * ratio * size, (g * ratio + 1) * size) for g in range(groups)], 0)


def _attention_transfer(source: dict, target: dict, src: str, name: str, shape: tuple[int, ...]) -> Expr | None:
    """The expression for tensor `name` (relative to the mixer) of a mixer that is initialised from an attention mixer at `src`."""
    heads, groups, size = source["heads"], source.get("head_groups", source["heads"]), source["head_size"]
    q, k, v, o = (Ref(f"{src}.{p}_proj.weight") for p in "qkvo")
    kind = target["type"]
    if kind == "mamba":
        inner, xb = target["d_inner"], target["d_xb"]
        if inner != heads * size or xb != groups * size:
            return None
        if name == "in_proj.weight":  # [z | x | B | C]
            return Concat([Init((inner, shape[1]), "normal", f"{src}.z", 0.02), v, k, q], 0)
        if name == "out_proj.weight":
            return o
    elif kind == "gdn":
        if (target["value_heads"], target["key_heads"], target["key_head_dim"], target["value_head_dim"]) != (heads, groups, size, size):
            return None
        if name == "in_proj_qkvz.weight":  # [q | k | v | z]
            return Concat([_first_of_groups(q, groups, heads, size), k, _repeat_groups(v, groups, heads, size),
                           Init((heads * size, shape[1]), "normal", f"{src}.z", 0.02)], 0)
        if name == "out_proj.weight":
            return o
    elif kind == "kda":
        if (target["heads"], target["head_dim"]) != (heads, size):
            return None
        if name == "q_proj.weight":
            return q
        if name == "k_proj.weight":
            return _repeat_groups(k, groups, heads, size)
        if name == "v_proj.weight":
            return _repeat_groups(v, groups, heads, size)
        if name == "o_proj.weight":
            return o
    return None


def _plan_mixer(plan: Plan, source_mixer: dict, target_mixer: dict, src: str, dst: str, target_shapes: dict, source_shapes: dict, scale: float) -> None:
    names = [n for n in target_shapes if n.startswith(dst + ".")]
    target_type, source_type = target_mixer.get("type", "attention"), source_mixer.get("type", "attention")
    if target_type == "stochastic":
        for sub_name, sub in target_mixer["mixers"].items():
            sub_dst = f"{dst}.mixers.{sub_name}"
            if source_type == "stochastic":
                main = source_mixer.get("main_mixer_name") or next(iter(source_mixer["mixers"]))
                origin = sub_name if sub_name in source_mixer["mixers"] else main
                _plan_mixer(plan, source_mixer["mixers"][origin], sub, f"{src}.mixers.{origin}", sub_dst, target_shapes, source_shapes, scale)
            else:
                _plan_mixer(plan, source_mixer, sub, src, sub_dst, target_shapes, source_shapes, scale)
        return
    if source_type == "stochastic":  # unwrap: the named (or main) sub-mixer carries on
        main = source_mixer.get("main_mixer_name") or next(iter(source_mixer["mixers"]))
        candidates = [n for n, m in source_mixer["mixers"].items() if m.get("type", "attention") == target_type]
        origin = main if (main in candidates or not candidates) else candidates[0]
        return _plan_mixer(plan, source_mixer["mixers"][origin], target_mixer, f"{src}.mixers.{origin}", dst, target_shapes, source_shapes, scale)
    mode = target_mixer.get(INIT_KEY, "transfer")
    for name in names:
        relative = name[len(dst) + 1:]
        shape = target_shapes[name][0]
        expr = None
        if mode == "transfer":
            if source_type == target_type:
                candidate = f"{src}.{relative}"
                if source_shapes.get(candidate, (None,))[0] == shape:
                    expr = Ref(candidate)
            elif source_type == "attention":
                expr = _attention_transfer(source_mixer, target_mixer, src, relative, shape)
        plan[name] = expr if expr is not None else _new_values(name, shape, scale)


def plan_surgery(source_state: dict, transition: dict) -> Plan:
    """source state x transition -> the plan that builds the target checkpoint's tensors from the source checkpoint's."""
    source_state = strip_init_fields(source_state)
    target_state = strip_init_fields(transition)
    source_shapes, target_shapes = _shapes(source_state), _shapes(target_state)
    scale = float(target_state.get("initializer_range", 0.02))
    source_blocks, target_blocks = block_configs(source_state), block_configs(transition)
    plan = Plan()
    for index, block in enumerate(target_blocks):
        dst = f"model.decoder.blocks.{index}.mixer"
        if index < len(source_blocks):
            _plan_mixer(plan, source_blocks[index]["mixer"], block["mixer"], dst, dst, target_shapes, source_shapes, scale)
    for name, (shape, _) in target_shapes.items():
        if name in plan:
            continue
        plan[name] = Ref(name) if source_shapes.get(name, (None,))[0] == shape else _new_values(name, shape, scale)
    return Plan({name: plan[name] for name in target_shapes})  # in the target model's own order


def apply_surgeries(state: dict, surgeries: list[dict]) -> tuple[dict, Plan]:
    """A chain of surgeries as (final state, one plan from the first state's tensors)."""
    current = strip_init_fields(state)
    plan = Plan({name: Ref(name) for name in _shapes(current)})
    for surgery in surgeries:
        transition = compose_configs(current, surgery)
        plan = compose_plans(plan, plan_surgery(current, transition))
        current = strip_init_fields(transition)  # `init: random` applies to the surgery that introduces a component only
    return current, plan


# ---------------------------------------------------------------------------------------------- files


class _LazyCheckpoint(typing.Mapping):
    """The tensors of a Hugging Face safetensors directory, opened on demand."""

    def __init__(self, path: pathlib.Path):
        import safetensors

        self._files = {}
        index = path / "model.safetensors.index.json"
        if index.exists():
            for name, file in json.loads(index.read_text())["weight_map"].items():
                self._files[name] = path / file
        else:
            for file in sorted(path.glob("*.safetensors")):
                with safetensors.safe_open(str(file), framework="pt") as f:
                    for name in f.keys():
                        self._files[name] = file

    def __getitem__(self, name):
        import safetensors

        with safetensors.safe_open(str(self._files[name]), framework="pt") as f:
            return f.get_tensor(name)

    def __iter__(self):
        return iter(self._files)

    def __len__(self):
        return len(self._files)


def convert_checkpoint(input_path, output_path, surgeries: list[dict], seed: int = 0, shard_bytes: int = 4 << 30) -> dict:
    """Apply `surgeries` to the Apriel2 text checkpoint at `input_path`; writes config.json, sharded safetensors with an index,
    the plan (`surgery_plan.json`) and the modelling files.  Returns the new configuration."""
    import safetensors.torch

    input_path, output_path = pathlib.Path(input_path), pathlib.Path(output_path)
    output_path.mkdir(parents=True, exist_ok=True)
    config = json.loads((input_path / "config.json").read_text())
    state, plan = apply_surgeries(config, surgeries)
    source = _LazyCheckpoint(input_path)
    missing = plan.source_keys() - set(source)
    if missing:
        raise KeyError(f"the plan needs tensors the input checkpoint does not have: {sorted(missing)[:8]}")
    dtype = getattr(torch, str(config.get("torch_dtype", config.get("dtype", "float32"))))
    weight_map, shard, size, count = {}, {}, 0, 0

    def flush():
        nonlocal shard, size, count
        if shard:
            file = f"model_{count}.safetensors"
            safetensors.torch.save_file(shard, str(output_path / file))
            weight_map.update({name: file for name in shard})
            shard, size, count = {}, 0, count + 1

    for name, tensor in plan.stream(source, seed):
        tensor = tensor.to(dtype) if tensor.is_floating_point() else tensor
        shard[name] = tensor
        size += tensor.numel() * tensor.element_size()
        if size >= shard_bytes:
            flush()
    flush()
    (output_path / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": weight_map}, indent=2))
    (output_path / "config.json").write_text(json.dumps(state, indent=2))
    (output_path / "surgery_plan.json").write_text(json.dumps(plan.to_dict(), indent=1))
    for extra in ("configuration_apriel2.py", "modeling_apriel2.py"):
        source_file = pathlib.Path(__file__).with_name(extra)
        if source_file.exists():
            (output_path / extra).write_text(source_file.read_text())
    return state


def main(argv=None) -> None:
    import yaml

    parser = argparse.ArgumentParser(description="Apply surgeries to an Apriel2 text checkpoint.")
    parser.add_argument("input")
    parser.add_argument("output")
    parser.add_argument("--surgery", action="append", default=[], help="YAML or JSON file with a partial configuration (repeatable: a chain)")
    parser.add_argument("--seed", type=int, default=0)
    parser.add_argument("--dry-run", action="store_true", help="print the plan summary and the target configuration, write nothing")
    args = parser.parse_args(argv)
    surgeries = [yaml.safe_load(pathlib.Path(p).read_text()) for p in args.surgery]
    if args.dry_run:
        state, plan = apply_surgeries(json.loads((pathlib.Path(args.input) / "config.json").read_text()), surgeries)
        print(plan.summary())
        print(json.dumps(state, indent=2))
        return
    convert_checkpoint(args.input, args.output, surgeries, args.seed)


if __name__ == "__main__":
    main()
