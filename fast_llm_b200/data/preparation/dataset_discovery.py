"""Build one blended dataset config for every prepared file under a directory tree.

Each directory becomes a blend of its files and sub-directories, weighted by token count, so the final mix samples every
token of the tree with equal probability.  Parity: `fast_llm/data/preparation/dataset_discovery/prepare.py:18-138`.
"""

import logging
import pathlib

import yaml

from fast_llm_b200.data.memmap import MemmapDataset

logger = logging.getLogger(__name__)


class DatasetDiscoveryPreparator:
    def __init__(self, config):
        self._config = config

    def run(self) -> None:
        root = pathlib.Path(self._config.directory)
        ignored = [(p if pathlib.Path(p).is_absolute() else root / p).resolve() for p in self._config.ignore_paths]
        found = self._scan(root, root, ignored)
        if found is None:
            raise ValueError(f"No .fast_llm_dataset file under {root}")
        config, tokens = found
        output = pathlib.Path(self._config.output)
        output.parent.mkdir(parents=True, exist_ok=True)
        output.write_text(yaml.safe_dump({"config": config, "metadata": {"num_tokens": tokens}}))
        logger.info(f"Wrote {output}: {tokens:,} tokens")

    def _scan(self, directory: pathlib.Path, root: pathlib.Path, ignored: list[pathlib.Path]):
        entries = []
        for path in sorted(directory.iterdir()):
            if any(path.resolve() == skip or skip in path.resolve().parents for skip in ignored):
                continue
            if path.is_dir():
                sub = self._scan(path, root, ignored)
                if sub is not None:
                    entries.append(sub)
            elif path.suffix == ".fast_llm_dataset":
                try:
                    tokens = int(MemmapDataset(path.stem, path).num_tokens)
                except Exception as e:  # unreadable or foreign file: skip, but say so
                    logger.warning(f"Skipping {path}: {e}")
                    continue
                if tokens > 0:
                    entries.append(({"type": "memmap", "path": str(path.resolve())}, tokens))
        if not entries:
            return None
        if len(entries) == 1:
            return entries[0]
        return ({"type": "blended", "name": str(directory.relative_to(root)) or root.name, "datasets": [e[0] for e in entries],
                 "weights": [e[1] for e in entries]}, sum(e[1] for e in entries))
