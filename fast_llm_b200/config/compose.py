"""Hydra-style composition without the hydra package: a `defaults` list that merges other YAML files of a config
directory, config-group selection from the command line, and the override grammar `key=value` / `+key=value` /
`++key=value` / `~key[=value]`.  Parity of behaviour: `fast_llm/engine/config_utils/runnable.py:155-178` (which delegates
to `hydra.compose`); only the subset of hydra that composing training configs needs is covered: no interpolation, no
sweeps, no packages other than the group's own key.
"""

import copy
import pathlib
import typing

import yaml


def _merge(base: dict, update: dict) -> dict:
    for key, value in update.items():
        if isinstance(value, dict) and isinstance(base.get(key), dict):
            _merge(base[key], value)
        else:
            base[key] = copy.deepcopy(value)
    return base


def _load(directory: pathlib.Path, name: str) -> dict:
    for suffix in ("", ".yaml", ".yml"):
        path = directory / f"{name}{suffix}"
        if path.is_file():
            return yaml.safe_load(path.read_text()) or {}
    raise FileNotFoundError(f"No config {name!r} under {directory}")


def _compose_file(directory: pathlib.Path, name: str, group_choices: dict[str, str], package: tuple[str, ...] = ()) -> dict:
    """Load `name`, resolve its `defaults` list depth-first; later entries win, `_self_` marks where the file's own keys go
    (at the end when absent)."""
    content = _load(directory, name)
    defaults = content.pop("defaults", [])
    result: dict = {}
    own_done = False

    def place(target: dict, path: tuple[str, ...], value: dict):
        for key in path:
            target = target.setdefault(key, {})
        _merge(target, value)

    for entry in defaults:
        if entry == "_self_":
            place(result, package, content)
            own_done = True
        elif isinstance(entry, str):
            _merge(result, _compose_file(directory, str(pathlib.PurePosixPath(name).parent / entry) if "/" in name else entry, group_choices))
        elif isinstance(entry, dict):
            for group, option in entry.items():
                group = group.removeprefix("optional ").removeprefix("override ").strip()
                option = group_choices.pop(group, option)
                if option is None or option == "null":
                    continue
                try:
                    chosen = _compose_file(directory, f"{group}/{option}", group_choices)
                except FileNotFoundError:
                    if str(next(iter(entry))).startswith("optional "):
                        continue
                    raise
                place(result, tuple(group.split("/")), chosen)
        else:
            raise ValueError(f"Unsupported entry in the defaults list of {name}: {entry!r}")
    if not own_done:
        place(result, package, content)
    return result


def compose_config(directory: pathlib.Path | None, name: str | None, base: dict, overrides: list[str]) -> tuple[dict, list[str]]:
    """Returns the composed config and the overrides that remain to be applied to it (group selections are consumed)."""
    if name is None:
        return copy.deepcopy(base), list(overrides)
    directory = pathlib.Path(directory)
    group_choices, remaining = {}, []
    for arg in overrides:
        key, _, value = arg.partition("=")
        if value and not key.startswith(("+", "~")) and (directory / key).is_dir():
            group_choices[key] = value
        else:
            remaining.append(arg)
    composed = _compose_file(directory, name, group_choices)
    if group_choices:
        raise ValueError(f"Config groups {sorted(group_choices)} were selected but do not appear in any defaults list")
    return composed, remaining


def apply_overrides(config: dict, overrides: typing.Iterable[str]) -> dict:
    """`a.b=v` changes an existing key, `+a.b=v` adds a new one, `++a.b=v` does either, `~a.b` (or `~a.b=v`) removes."""
    for arg in overrides:
        mode = "set"
        if arg.startswith("++"):
            mode, arg = "force", arg[2:]
        elif arg.startswith("+"):
            mode, arg = "add", arg[1:]
        elif arg.startswith("~"):
            mode, arg = "delete", arg[1:]
        key, has_value, raw = arg.partition("=")
        if not has_value and mode != "delete":
            raise ValueError(f"Cannot parse override {arg!r}: expected key=value")
        path = key.split(".")
        node = config
        for part in path[:-1]:
            if part not in node or not isinstance(node[part], dict):
                if mode in ("set", "delete"):
                    raise KeyError(f"Override {arg!r}: {part!r} does not exist (use +{key}=... to add it)")
                node[part] = {}
            node = node[part]
        leaf = path[-1]
        if mode == "delete":
            if leaf not in node:
                raise KeyError(f"Override ~{key}: key does not exist")
            if has_value and node[leaf] != yaml.safe_load(raw):
                raise ValueError(f"Override ~{key}={raw}: current value is {node[leaf]!r}")
            del node[leaf]
            continue
        if mode == "set" and leaf not in node:
            raise KeyError(f"Override {arg!r}: key does not exist (use +{key}={raw} to add it)")
        if mode == "add" and leaf in node:
            raise KeyError(f"Override +{arg}: key already exists (use ++{key}={raw} to change it)")
        node[leaf] = yaml.safe_load(raw)
    return config
