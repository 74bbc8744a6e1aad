"""Streaming dataset: documents arrive over a Redis stream (produced by RL rollout workers) instead of from disk.

Wire format of one stream entry (compatible with the reference producer): `tokens` = int64 bytes,
`old_log_probabilities` = float32 bytes (optional), `data` = JSON with `loss_masking_spans`, `chosen_span`,
`rejected_span`, `advantage`, `reward` (all optional).  The consumer group makes every entry reach exactly one rank.
Samples are built by packing whole documents, in arrival order, until the next one no longer fits.
Parity: `fast_llm/data/dataset/streaming.py:23-230`, `fast_llm/data/dataset/config.py` (StreamingDatasetConfig).
"""

import json
import time
import typing

import numpy as np
import torch

from fast_llm_b200.data.document import LanguageModelDocument

REDIS_DATA_STREAM = "fast_llm_streaming"
REDIS_GROUP_NAME = "fast_llm_group"


def encode_document(tokens, *, old_log_probabilities=None, loss_masking_spans=None, chosen_span=None, rejected_span=None,
                    advantage: float | None = None, reward: float | None = None) -> dict[str, bytes | str]:
    """Producer side: one stream entry."""
    message: dict[str, bytes | str] = {"tokens": np.asarray(tokens, dtype=np.int64).tobytes()}
    if old_log_probabilities is not None:
        message["old_log_probabilities"] = np.asarray(old_log_probabilities, dtype=np.float32).tobytes()
    data = {key: value for key, value in (("loss_masking_spans", loss_masking_spans), ("chosen_span", chosen_span),
                                           ("rejected_span", rejected_span), ("advantage", advantage), ("reward", reward)) if value is not None}
    if data:
        message["data"] = json.dumps(data)
    return message


def decode_document(message: dict) -> LanguageModelDocument:
    fields: dict[str, typing.Any] = {}
    for key, value in message.items():
        key = key.decode() if isinstance(key, bytes) else key
        if key == "data":
            fields.update(json.loads(value))
        else:
            fields[key] = value

    def as_tensor(value, dtype):
        if value is None:
            return None
        if isinstance(value, (bytes, bytearray)):
            return torch.from_numpy(np.frombuffer(value, dtype=dtype).copy())
        return torch.tensor(value, dtype=torch.from_numpy(np.zeros(0, dtype=dtype)).dtype)

    tokens = as_tensor(fields["tokens"], np.int64)
    old = as_tensor(fields.get("old_log_probabilities"), np.float32)
    if old is not None and len(old) != len(tokens):
        raise ValueError(f"old_log_probabilities has {len(old)} entries for {len(tokens)} tokens")
    advantage = fields.get("advantage")
    spans = fields.get("loss_masking_spans")
    return LanguageModelDocument(
        tokens=tokens, loss_masking_spans=[tuple(s) for s in spans] if spans else None,
        chosen_span=tuple(fields["chosen_span"]) if fields.get("chosen_span") else None,
        rejected_span=tuple(fields["rejected_span"]) if fields.get("rejected_span") else None,
        advantages=None if advantage is None else torch.full((len(tokens),), float(advantage)),
        old_log_probabilities=old)


class RedisStreamingDataset:
    """Sequential sampled dataset over a Redis stream; `client` can be injected (tests use an in-memory stand-in)."""

    requires_broadcast = True  # only one rank of a model-parallel group reads; the batch is broadcast to the others

    def __init__(self, config, sampling, client=None):
        self._config, self._sampling = config, sampling
        self._client = client
        self._carry: LanguageModelDocument | None = None
        self._next_index = 0
        self._group_ready = False
        self.name = f"redis[{config.host}:{config.port}]({REDIS_DATA_STREAM}|{REDIS_GROUP_NAME})"

    def __len__(self) -> int:
        return self._sampling.num_samples or 2**62

    def _ensure_group(self):
        if self._client is None:
            self._client = self._config.get_client()
        if not self._group_ready:
            try:
                self._client.xgroup_create(name=REDIS_DATA_STREAM, groupname=REDIS_GROUP_NAME, id="0", mkstream=True)
            except Exception as e:  # the group already exists
                if "BUSYGROUP" not in str(e):
                    raise
            self._group_ready = True

    def _read_document(self) -> LanguageModelDocument:
        self._ensure_group()
        start = time.time()
        while True:
            messages = self._client.xreadgroup(groupname=REDIS_GROUP_NAME, consumername=f"fast_llm_consumer_{self._sampling.rank}",
                                               streams={REDIS_DATA_STREAM: ">"}, count=1, block=1000, noack=True)
            for _, entries in messages or ():
                for _, message in entries:
                    return decode_document(message)
            waited = time.time() - start
            if waited > self._config.timeout:
                raise TimeoutError(f"No document received after {waited:.0f} seconds")

    def __getitem__(self, index: int) -> list[LanguageModelDocument]:
        if index < self._next_index:
            raise IndexError(f"A stream is read in order: sample {index} was asked for after sample {self._next_index - 1}")
        self._next_index = index + 1  # batch-data ranks ask for every n-th index: each is its own consumer of the stream
        size = self._sampling.sample_size
        documents, used = [], 0
        while True:
            document = self._carry if self._carry is not None else self._read_document()
            self._carry = None
            if len(document) > size:
                document = document.crop(0, size)
            if used + len(document) > size:
                self._carry = document  # opens the next sample
                return documents
            documents.append(document)
            used += len(document)
            if used == size:
                return documents
