"""Tokenizer wrapper (Hugging Face `tokenizers` / `transformers`), with the span-aware and chat-template helpers the
data preparation needs.

`tokenize(text, begin, end)` adds the beginning/end-of-document tokens explicitly (never the tokenizer's own special-token
logic), `tokenize_with_spans` cuts the text at span boundaries so character spans map exactly onto token spans,
`tokenize_chat` renders a conversation with the chat template and returns the loss-masking spans of everything that is
not an assistant turn.  Parity: `fast_llm/data/preparation/tokenizer.py:18-331`.
"""

import bisect
import functools
import pathlib

import numpy as np
import torch

from fast_llm_b200.utils import Assert


class Tokenizer:
    def __init__(self, config):
        self._config = config
        path = pathlib.Path(config.path)
        self.tokenizer = self._load(path, config.trust_remote_code)
        if config.bos_token is not None:
            self.tokenizer.bos_token = config.bos_token
        self.eod_id = self.tokenizer.eos_token_id
        self.bod_id = self.tokenizer.bos_token_id

    @staticmethod
    def _load(path: pathlib.Path, trust_remote_code: bool):
        import transformers

        if path.is_file() and path.suffix == ".json":  # a bare `tokenizer.json`
            return transformers.PreTrainedTokenizerFast(tokenizer_file=str(path))
        return transformers.AutoTokenizer.from_pretrained(str(path), errors="replace", max_len=None, trust_remote_code=trust_remote_code, use_fast=True)

    # ---- vocabulary
    @functools.cached_property
    def _tokenizer_vocab_size(self) -> int:
        return len(self.tokenizer)

    @functools.cached_property
    def vocab_size(self) -> int:
        limit = self._config.max_vocab_size
        return self._tokenizer_vocab_size if limit is None else min(self._tokenizer_vocab_size, limit)

    @property
    def vocab(self) -> dict[str, int]:
        return self.tokenizer.get_vocab()

    @functools.cached_property
    def inv_vocab(self) -> dict[int, str]:
        return {index: token for token, index in self.vocab.items()}

    @property
    def eod(self) -> int:
        return self.eod_id

    # ---- text -> tokens
    def tokenize(self, text: str, begin: bool = True, end: bool = True, data_type: torch.dtype = torch.int64) -> torch.Tensor:
        tokens = self.tokenizer.encode(text, add_special_tokens=False)
        if begin:
            Assert.not_none(self.bod_id)
            tokens = [self.bod_id, *tokens]
        if end:
            Assert.not_none(self.eod_id)
            tokens = [*tokens, self.eod_id]
        out = torch.tensor(tokens, dtype=torch.int64)
        if self._config.max_vocab_size is not None:
            out = out % self._config.max_vocab_size
        return out.to(data_type)

    def tokenize_with_splits(self, text: str, begin: bool = True, end: bool = True, *, text_splits: list[int],
                             data_type: torch.dtype = torch.int64) -> tuple[torch.Tensor, list[int]]:
        """Tokenize piecewise between the (character) split points; returns tokens and the token index of each split,
        in the order the splits were given."""
        if not text_splits:
            return self.tokenize(text, begin, end, data_type), []
        order = np.argsort(text_splits, kind="stable")
        edges = [0, *(text_splits[i] for i in order), len(text)]
        pieces, token_splits, total = [], [], 0
        for i, (lo, hi) in enumerate(zip(edges[:-1], edges[1:])):
            piece = self.tokenize(text[lo:hi], begin and i == 0, end and i == len(edges) - 2, data_type)
            pieces.append(piece)
            total += len(piece)
            token_splits.append(total)
        restored = np.empty(len(order), dtype=np.int64)
        restored[order] = token_splits[:-1]
        return torch.cat(pieces), restored.tolist()

    def tokenize_with_spans(self, text: str, begin: bool = True, end: bool = True, *, text_spans: list[tuple[int, int]],
                            data_type: torch.dtype = torch.int64) -> tuple[torch.Tensor, list[tuple[int, int]]]:
        if not text_spans:
            return self.tokenize(text, begin, end, data_type), []
        tokens, splits = self.tokenize_with_splits(text, begin, end, text_splits=[edge for span in text_spans for edge in span], data_type=data_type)
        return tokens, list(zip(splits[::2], splits[1::2]))

    # ---- tokens -> text
    def _strip(self, tokens, begin: bool, end: bool):
        if begin:
            Assert.eq(int(tokens[0]), self.bod_id)
            tokens = tokens[1:]
        if end:
            Assert.eq(int(tokens[-1]), self.eod_id)
            tokens = tokens[:-1]
        return tokens

    def detokenize(self, tokens, begin: bool = False, end: bool = False) -> str:
        tokens = self._strip(tokens, begin, end)
        if torch.is_tensor(tokens) or isinstance(tokens, np.ndarray):
            tokens = tokens.tolist()
        return self.tokenizer.decode(tokens)

    def detokenize_with_splits(self, tokens, begin: bool = False, end: bool = False, *, token_splits: list[int]) -> tuple[str, list[int]]:
        if not token_splits:
            return self.detokenize(tokens, begin, end), []
        Assert.eq(sorted(token_splits), list(token_splits))
        tokens = self._strip(tokens, begin, end)
        edges = [0, *(split - int(begin) for split in token_splits), len(tokens)]
        texts, text_splits, total = [], [], 0
        for lo, hi in zip(edges[:-1], edges[1:]):
            texts.append(self.detokenize(tokens[lo:hi]))
            total += len(texts[-1])
            text_splits.append(total)
        return "".join(texts), text_splits[:-1]

    def detokenize_with_spans(self, tokens, begin: bool = False, end: bool = False, *, token_spans: list[tuple[int, int]]) -> tuple[str, list[tuple[int, int]]]:
        if not token_spans:
            return self.detokenize(tokens, begin, end), []
        text, splits = self.detokenize_with_splits(tokens, begin, end, token_splits=[edge for span in token_spans for edge in span])
        return text, list(zip(splits[::2], splits[1::2]))

    # ---- chat
    def validate_chat_template(self) -> None:
        template = getattr(self.tokenizer, "chat_template", None)
        if template is None:
            raise ValueError("The tokenizer has no chat template; conversations cannot be tokenized")
        if "generation" not in template:
            raise ValueError("The chat template lacks `{% generation %}` markers, needed to tell assistant tokens from the rest")

    def tokenize_chat(self, messages: list[dict[str, str]], begin: bool = True, end: bool = True,
                      data_type: torch.dtype = torch.int64) -> tuple[torch.Tensor, list[tuple[int, int]]]:
        """Render with the chat template; returns tokens and loss-masking spans covering every non-assistant token."""
        encoded = self.tokenizer.apply_chat_template(messages, tokenize=True, return_assistant_tokens_mask=True, return_dict=True,
                                                     add_generation_prompt=False)
        tokens = list(encoded["input_ids"])
        train_mask = [bool(m) for m in encoded["assistant_masks"]]
        if begin and (not tokens or tokens[0] != self.bod_id):
            tokens, train_mask = [self.bod_id, *tokens], [False, *train_mask]
        if end and (not tokens or tokens[-1] != self.eod_id):
            tokens, train_mask = [*tokens, self.eod_id], [*train_mask, True]
        return torch.tensor(tokens, dtype=data_type), train_mask_to_loss_spans(train_mask)


def train_mask_to_loss_spans(train_mask: list[bool]) -> list[tuple[int, int]]:
    """Maximal runs of `False` (tokens excluded from the loss) as half-open spans."""
    spans, start = [], None
    for i, keep in enumerate(train_mask):
        if not keep and start is None:
            start = i
        elif keep and start is not None:
            spans.append((start, i))
            start = None
    if start is not None:
        spans.append((start, len(train_mask)))
    return spans
