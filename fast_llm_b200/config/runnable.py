"""Command-line entry for configs that can run: `fast-llm <sub-command...> [-c file.yaml] [key.sub=value ...]`.

Parity: `fast_llm/engine/config_utils/runnable.py:36-238` — leading arguments select registered sub-classes, a YAML
file gives defaults, dotted `key=value` arguments override them, `-v/--validate` stops after validation.
"""

import argparse
import logging
import pathlib
import sys
import typing
import urllib.parse

import yaml

from fast_llm_b200.config.core import Config, FieldVerboseLevel, NoAutoValidate, config_class

logger = logging.getLogger(__name__)


@config_class(registry=True)
class RunnableConfig(Config):
    _ALLOWED_CONFIG_HOSTS: typing.ClassVar[frozenset] = frozenset({"github.com", "raw.githubusercontent.com", "api.github.com"})

    @classmethod
    def parse_and_run(cls, args: list[str] | None = None):
        args = list(sys.argv[1:] if args is None else args)
        if args and not args[0].startswith("-") and "=" not in args[0]:
            try:
                sub = cls.get_subclass(args[0])
            except KeyError:
                sub = None
            if sub is not None and sub is not cls:
                return sub.parse_and_run(args[1:])
            if sub is None and cls._abstract:
                raise KeyError(f"Unknown sub-command {args[0]!r} for {cls.__name__}")
        parsed, unparsed = cls._get_parser().parse_known_args(args)
        with NoAutoValidate():
            config = cls._from_parsed_args(parsed, unparsed)
        try:
            config.configure_logging()
            config.validate()
            if not parsed.do_run:
                return config
            runnable = config._get_runnable()
        finally:
            pass
        config._show(parsed.verbose)
        return runnable()

    @classmethod
    def _get_parser(cls) -> argparse.ArgumentParser:
        parser = argparse.ArgumentParser(description=cls.__doc__)
        parser.add_argument("-v", "--validate", dest="do_run", action="store_false", help="Validate the config without running.")
        parser.add_argument("--verbose", type=int, help="Verbosity of the config printout.", default=FieldVerboseLevel.core)
        parser.add_argument("-c", "--config", type=str, help="YAML config file (path or allow-listed https URL).")
        parser.add_argument("--hydra", action="store_true", help="Hydra override syntax for the command-line updates: key=value, +key=value, ++key=value, ~key.")
        parser.add_argument("--hydra-path", type=pathlib.Path, default=None, help="Directory of composable YAML configs (implies --hydra).")
        parser.add_argument("--hydra-config", type=str, default=None, help="Base config inside --hydra-path (replaces --config); its `defaults` list is composed.")
        parser.add_argument("--config_auth_token_file", type=pathlib.Path, default=None)
        parser.add_argument("--trust-remote-code", action="store_true", help="Allow Hugging Face remote code when loading tokenizers/models.")
        return parser

    @classmethod
    def _from_parsed_args(cls, parsed: argparse.Namespace, unparsed: list[str]):
        default = cls._load_default_config_dict(parsed)
        if parsed.hydra or parsed.hydra_path is not None or parsed.hydra_config is not None:
            from fast_llm_b200.config.compose import apply_overrides, compose_config

            if parsed.hydra_config is not None:
                if default:
                    raise ValueError("--hydra-config replaces --config: give only one of them")
                if parsed.hydra_path is None:
                    raise ValueError("--hydra-config needs --hydra-path")
            default, remaining = compose_config(parsed.hydra_path, parsed.hydra_config, default, unparsed)
            return cls.from_dict(apply_overrides(default, remaining), {})
        updates = cls._parse_updates(unparsed)
        return cls.from_dict(default, updates)

    def configure_logging(self) -> None:
        logging.basicConfig(level=logging.INFO, format="%(asctime)s %(message)s", force=False)

    def _get_runnable(self) -> typing.Callable[[], None]:
        return self.run

    def run(self) -> None:
        raise NotImplementedError(f"{type(self).__name__} has nothing to run")

    def _show(self, verbose: int | None = FieldVerboseLevel.core, *, log_fn=logger.info, title: str | None = None):
        return self.to_logs(verbose=verbose, log_fn=log_fn, title=title)

    @classmethod
    def _load_default_config_dict(cls, parsed: argparse.Namespace) -> dict:
        if parsed.config is None:
            return {}
        url = urllib.parse.urlparse(parsed.config)
        if url.scheme == "https":
            if url.hostname not in cls._ALLOWED_CONFIG_HOSTS:
                raise ValueError(f"Config host {url.hostname} is not allow-listed ({sorted(cls._ALLOWED_CONFIG_HOSTS)})")
            import requests

            headers = {"Accept": "application/vnd.github.v3.raw"}
            if parsed.config_auth_token_file is not None:
                headers["Authorization"] = f"token {parsed.config_auth_token_file.read_text().strip()}"
            response = requests.get(parsed.config, headers=headers, timeout=60)
            response.raise_for_status()
            return yaml.safe_load(response.text) or {}
        with open(parsed.config) as f:
            return yaml.safe_load(f) or {}

    @classmethod
    def _parse_updates(cls, unparsed: list[str]) -> dict:
        updates = {}
        for arg in unparsed:
            if "=" not in arg:
                raise ValueError(f"Cannot parse argument {arg!r}: expected key.sub=value")
            key, value = arg.split("=", 1)
            key = key.lstrip("-")
            updates[tuple(key.split("."))] = yaml.safe_load(value)
        return updates
