"""Generate the configuration reference: one Markdown page per config class plus an index.

    python -m fast_llm_b200.tools.generate_config_docs [output_dir]

Every class built with `@config_class` in the package is imported, its user-facing fields are listed with type, default,
importance hint and description, its registered `type:` names are shown, and pages link to the classes they nest and to
the classes that use them.  Parity: `tools/generate_config_docs.py` (class pages, back references, per-package index).
"""

import importlib
import pathlib
import pkgutil
import sys
import typing

from fast_llm_b200.config import Config, FieldHint
from fast_llm_b200.config.core import MISSING, _config_class_of

EXCLUDED_HINTS = {FieldHint.derived, FieldHint.setup, FieldHint.testing}


def import_all_modules(package: str = "fast_llm_b200") -> None:
    root = importlib.import_module(package)
    for module in pkgutil.walk_packages(root.__path__, prefix=package + "."):
        if ".csrc" in module.name or module.name.endswith("__main__"):
            continue
        try:
            importlib.import_module(module.name)
        except Exception as e:  # optional dependencies
            print(f"skipping {module.name}: {type(e).__name__}: {e}", file=sys.stderr)


def all_config_classes() -> list[type[Config]]:
    seen, stack = [], [Config]
    while stack:
        cls = stack.pop()
        for sub in cls.__subclasses__():
            if sub not in seen and sub.__module__.startswith("fast_llm_b200"):
                seen.append(sub)
                stack.append(sub)
            elif sub not in seen:
                stack.append(sub)
    return sorted(seen, key=lambda c: (c.__module__, c.__name__))


def user_fields(cls: type[Config]) -> dict:
    return {name: field for name, field in cls.fields().items()
            if not name.startswith("_") and name != "type" and field.init and field.hint not in EXCLUDED_HINTS}


def nested_config_types(annotation) -> list[type[Config]]:
    found = []
    direct = _config_class_of(annotation)
    if direct is not None:
        found.append(direct)
    for arg in typing.get_args(annotation):
        found += nested_config_types(arg)
    return found


def page_path(cls: type[Config]) -> pathlib.Path:
    return pathlib.Path(*cls.__module__.split(".")[1:]) / f"{cls.__name__}.md"


def _link(from_cls, to_cls) -> str:
    import os

    return f"[{to_cls.__name__}]({os.path.relpath(page_path(to_cls), page_path(from_cls).parent)})"


def render_type(cls, annotation) -> str:
    nested = nested_config_types(annotation)
    text = getattr(annotation, "__name__", None) if isinstance(annotation, type) else None
    text = text or str(annotation).replace("typing.", "").replace("fast_llm_b200.", "")
    for sub in nested:
        text = text.replace(f"{sub.__module__}.{sub.__name__}".replace("fast_llm_b200.", ""), sub.__name__)
        text = text.replace(sub.__name__, _link(cls, sub), 1)
    return text.replace("|", "\\|")


def render_default(field) -> str:
    if field.default is not MISSING:
        value = field.default
        return f"`{value.value if hasattr(value, 'value') and not isinstance(value, (int, float)) else value!r}`"
    if field.default_factory is not MISSING:
        try:
            return f"`{field.default_factory()!r}`"
        except Exception:
            return "*(built)*"
    return "*(sub-config defaults)*"


def render_class(cls: type[Config], back_references: dict) -> str:
    hints = typing.get_type_hints(cls)
    lines = [f"# {cls.__name__}", "", f"Module: `{cls.__module__}`", ""]
    doc = (cls.__doc__ or "").strip()
    if doc and not doc.startswith(cls.__name__ + "("):
        lines += [doc, ""]
    names = {base.__name__: name for base, name in getattr(cls, "_dynamic_type_names", {}).items()}
    if names:
        lines += ["Selected with " + ", ".join(f"`type: {name}` (as a `{base}`)" for base, name in names.items()) + ".", ""]
    registry = cls.__dict__.get("_registry")
    if registry:
        lines += ["Registered variants: " + ", ".join(f"`{name}` -> {_link(cls, sub)}" for name, sub in sorted(registry.items())), ""]
    fields = user_fields(cls)
    if fields:
        lines += ["| Field | Type | Default | Hint | Description |", "|---|---|---|---|---|"]
        for name, field in fields.items():
            description = " ".join(x for x in (field.desc, field.doc) if x) or ""
            lines.append(f"| `{name}` | {render_type(cls, hints.get(name, typing.Any))} | {render_default(field)} | {field.hint.value} | {description} |")
        lines.append("")
    else:
        lines += ["*No user-facing fields.*", ""]
    users = back_references.get(cls, [])
    if users:
        lines += ["Used by: " + ", ".join(f"{_link(cls, user)}.`{field}`" for user, field in users), ""]
    return "\n".join(lines)


def generate(output_dir: pathlib.Path) -> int:
    import fast_llm_b200.models.auto  # noqa: F401

    import_all_modules()
    classes = all_config_classes()
    back_references: dict = {}
    for cls in classes:
        try:
            hints = typing.get_type_hints(cls)
        except Exception:
            continue
        for name in user_fields(cls):
            for nested in nested_config_types(hints.get(name)):
                back_references.setdefault(nested, []).append((cls, name))
    index = ["# Configuration reference", "", f"{len(classes)} configuration classes.", ""]
    current = None
    for cls in classes:
        path = output_dir / page_path(cls)
        path.parent.mkdir(parents=True, exist_ok=True)
        try:
            path.write_text(render_class(cls, back_references))
        except Exception as e:
            print(f"failed on {cls.__name__}: {e}", file=sys.stderr)
            continue
        if cls.__module__ != current:
            current = cls.__module__
            index += ["", f"## `{current}`", ""]
        summary = (cls.__doc__ or "").strip().split("\n")[0]
        index.append(f"- [{cls.__name__}]({page_path(cls)})" + (f": {summary}" if summary and not summary.startswith(cls.__name__ + "(") else ""))
    (output_dir / "index.md").write_text("\n".join(index) + "\n")
    return len(classes)


def main(argv: list[str] | None = None) -> None:
    argv = sys.argv[1:] if argv is None else argv
    output = pathlib.Path(argv[0]) if argv else pathlib.Path("docs/reference/configuration")
    count = generate(output)
    print(f"wrote {count} pages under {output}")


if __name__ == "__main__":
    main()
