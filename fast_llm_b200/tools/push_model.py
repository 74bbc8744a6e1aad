"""Publish a run's exported checkpoints to the Hugging Face hub, one commit per checkpoint.

    python -m fast_llm_b200.tools.push_model experiment_dir=... repo_name=org/model model_type=mistral tokenizer_path=.../tokenizer.json

Every numbered directory under `<experiment_dir>/export/<format>/` (or `<experiment_dir>/export/`) that has no commit yet
(commit messages are the iteration numbers) is converted to the requested Hugging Face format when it is not one
already, staged together with the tokenizer files, and uploaded.  The hub client is created lazily and can be injected,
which is how the selection / staging logic is tested without network access.  Parity: `tools/push_model.py`.
"""

import logging
import os
import pathlib
import shutil
import typing

from fast_llm_b200.config import Field, FieldHint, config_class
from fast_llm_b200.config.runnable import RunnableConfig

logger = logging.getLogger(__name__)

OTHER_TOKENIZER_FILES = ("special_tokens_map.json", "tokenizer_config.json", "vocab.json", "merges.txt", "chat_template.jinja")


@config_class(dynamic_type={RunnableConfig: "push_model"})
class PushConfig(RunnableConfig):
    _abstract: typing.ClassVar[bool] = False
    experiment_dir: pathlib.Path = Field(default=None, desc="Experiment directory of the training run.", hint=FieldHint.core)
    repo_name: str = Field(default=None, desc="Hub repository (`organisation/name`).", hint=FieldHint.core)
    model_type: str = Field(default=None, desc="Hugging Face format of the uploaded checkpoints (llama, mistral, ...).", hint=FieldHint.core)
    tokenizer_path: pathlib.Path = Field(default=None, desc="`tokenizer.json` to ship with every checkpoint.", hint=FieldHint.core)
    model_class: str = Field(default="gpt", desc="Model family of the run.", hint=FieldHint.optional)
    tmp_checkpoint_dir: pathlib.Path | None = Field(default=None, desc="Staging directory (default: `<experiment_dir>/export_tmp`).", hint=FieldHint.optional)
    use_cpu: bool = Field(default=False, desc="Convert on the CPU.", hint=FieldHint.optional)
    private: bool = Field(default=True, desc="Create the repository as private.", hint=FieldHint.optional)

    def _validate(self):
        if self.tmp_checkpoint_dir is None and self.experiment_dir is not None:
            self.tmp_checkpoint_dir = pathlib.Path(self.experiment_dir) / "export_tmp"
        super()._validate()

    # ---- pieces (separately testable)
    @staticmethod
    def iteration_of(name: str) -> int | None:
        return int(name) if name.isdigit() and str(int(name)) == name else None

    def committed_iterations(self, api) -> set[int]:
        done = set()
        for commit in api.list_repo_commits(self.repo_name):
            number = self.iteration_of(commit.title.strip())
            if number is not None:
                done.add(number)
        return done

    def pending_checkpoints(self, committed: set[int]) -> list[tuple[int, pathlib.Path]]:
        export = pathlib.Path(self.experiment_dir) / "export"
        roots = [export, *(p for p in export.glob("*") if p.is_dir() and self.iteration_of(p.name) is None)]
        found = {}
        for root in roots:
            for path in root.glob("*"):
                number = self.iteration_of(path.name)
                if path.is_dir() and number is not None and number not in committed and (path / "ok").exists():
                    found.setdefault(number, path)
        return sorted(found.items())

    def stage(self, checkpoint: pathlib.Path) -> pathlib.Path:
        """Make `tmp_checkpoint_dir` hold exactly this checkpoint in the Hugging Face format plus the tokenizer."""
        staging = pathlib.Path(self.tmp_checkpoint_dir)
        staging.mkdir(parents=True, exist_ok=True)
        source = checkpoint
        if not (checkpoint / "config.json").exists():  # a native checkpoint: convert first
            from fast_llm_b200.engine.checkpoint.convert import ConvertConfig

            source = checkpoint.with_name(checkpoint.name + "_hf")
            if not (source / "ok").exists():
                convert = ConvertConfig.from_dict({"input": {"path": str(checkpoint), "format": "distributed" if (checkpoint / "rank_0.safetensors").exists() else "fast_llm"},
                                                   "output": {"path": str(source), "format": self.model_type}, "use_cpu": self.use_cpu, "model": self.model_class})
                convert.validate()
                convert.run()
        for file in source.iterdir():
            if file.name == "ok" or not file.is_file():
                continue
            target = staging / file.name
            target.unlink(missing_ok=True)
            try:
                target.hardlink_to(file)
            except OSError:
                shutil.copy(file, target)
        tokenizer = pathlib.Path(self.tokenizer_path)
        assert tokenizer.exists() and tokenizer.suffix == ".json", tokenizer
        shutil.copy(tokenizer, staging / "tokenizer.json")
        for name in OTHER_TOKENIZER_FILES:
            if tokenizer.with_name(name).exists():
                shutil.copy(tokenizer.with_name(name), staging / name)
        if (checkpoint / "metadata.yaml").exists():
            shutil.copy(checkpoint / "metadata.yaml", staging / "metadata.yaml")
        return staging

    def _api(self):
        import huggingface_hub

        token_path = os.environ.get("HUGGINGFACE_API_KEY_PATH")
        token = pathlib.Path(token_path).read_text().strip() if token_path else None
        return huggingface_hub.HfApi(token=token)

    def run(self, api=None) -> list[int]:
        api = api or self._api()
        api.create_repo(self.repo_name, private=self.private, exist_ok=True)
        pushed = []
        for number, checkpoint in self.pending_checkpoints(self.committed_iterations(api)):
            staging = self.stage(checkpoint)
            logger.info(f"Pushing iteration {number} to {self.repo_name}")
            api.upload_folder(folder_path=str(staging), repo_id=self.repo_name, commit_message=str(number))
            pushed.append(number)
        if self.tmp_checkpoint_dir is not None and pathlib.Path(self.tmp_checkpoint_dir).exists():
            shutil.rmtree(self.tmp_checkpoint_dir)
        return pushed


if __name__ == "__main__":
    PushConfig.parse_and_run()
