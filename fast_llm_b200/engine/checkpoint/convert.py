"""`fast-llm convert <model> input.format=... input.path=... output.format=... output.path=...`

Loads a checkpoint in one format and writes it in another, on one process (CPU or GPU), optionally a few stages at a
time (`layers_per_step`) so models larger than memory can be converted.  Parity: `fast_llm/engine/checkpoint/convert.py:19-162`.
"""

import json
import logging
import math
import pathlib

from fast_llm_b200.config import Field, FieldHint, config_class
from fast_llm_b200.config.runnable import RunnableConfig
from fast_llm_b200.engine.checkpoint.config import CheckpointLoadConfig, CheckpointSaveConfig
from fast_llm_b200.engine.multi_stage.config import FastLLMModelConfig, StageMode

logger = logging.getLogger(__name__)


@config_class(dynamic_type={RunnableConfig: "convert"})
class ConvertConfig(RunnableConfig):
    input: CheckpointLoadConfig = Field(desc="Checkpoint to read.")
    output: CheckpointSaveConfig = Field(desc="Checkpoint to write.")
    use_cpu: bool = Field(default=False, desc="Convert on the CPU.")
    exist_ok: bool = Field(default=False, desc="Overwrite an existing output directory.")
    layers_per_step: int | None = Field(default=None, desc="Convert this many layers at a time.")
    model: type[FastLLMModelConfig] = Field(default=None, desc="Model family.")

    @classmethod
    def _get_parser(cls):
        parser = super()._get_parser()
        parser.add_argument("model_type", help="Model family (for example gpt).")
        return parser

    @classmethod
    def _from_parsed_args(cls, parsed, unparsed):
        config = super()._from_parsed_args(parsed, unparsed)
        config.model = parsed.model_type
        return config

    def _validate(self):
        assert self.model is not None, "model type is required"
        if isinstance(self.model, str):
            self.model = FastLLMModelConfig.__fast_llm_from_name__(self.model)
        self.input.validate()
        self.output.validate()
        self.input.setup(self.model)
        self.output.setup(self.model)
        super()._validate()

    def _convert_model_partial(self, model_class, output: CheckpointSaveConfig, stage_filter: set | None = None):
        logger.info(f"Loading {self.input.format.name} checkpoint from {self.input.path}")
        model = model_class.from_pretrained(self.input, mode=StageMode.weights, use_cpu=self.use_cpu, stage_filter=stage_filter)
        logger.info(f"Saving {output.format.name} checkpoint to {output.path}")
        pathlib.Path(output.path).mkdir(parents=True, exist_ok=self.exist_ok or stage_filter is not None)
        model.save_checkpoint(output)
        (pathlib.Path(output.path) / "ok").touch()
        return model

    def run(self):
        model_class = self.model.get_model_class()
        output_path = pathlib.Path(self.output.path)
        if (output_path / "ok").exists() and not self.exist_ok:
            raise FileExistsError(f"Output {output_path} already holds a converted checkpoint (pass exist_ok=true to overwrite)")
        if self.layers_per_step is None:
            self._convert_model_partial(model_class, self.output)
            return
        # staged conversion: convert groups of stages into sub-directories, then merge their indexes
        metadata = self.model.load_metadata(self.input)
        probe = model_class(self.model.from_dict(metadata.config), verbose=False)
        num_stages = len(probe.stages)
        weight_map = {}
        steps = math.ceil(num_stages / self.layers_per_step)
        for step in range(steps):
            stages = set(range(step * self.layers_per_step, min((step + 1) * self.layers_per_step, num_stages)))
            part = self.output.to_copy({"path": str(output_path / str(step))})
            part.validate()
            part.setup(self.model)
            self._convert_model_partial(model_class, part, stages)
            index_file = output_path / str(step) / "model.safetensors.index.json"
            if index_file.exists():
                for name, file in json.loads(index_file.read_text())["weight_map"].items():
                    weight_map[name] = f"{step}/{file}"
                if step == 0:
                    for extra in ("config.json",):
                        if (output_path / "0" / extra).exists():
                            (output_path / extra).write_text((output_path / "0" / extra).read_text())
        if weight_map:
            (output_path / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": weight_map}, indent=2))
        (output_path / "ok").touch()
