"""Fill-in-the-middle augmentation of sampled token sequences.

Every document of a sample (split at end-of-document tokens) is, with probability `rate`, cut at two random character
positions into prefix / middle / suffix and re-emitted as `<prefix> p <suffix> s <middle> m` (PSM) or
`<prefix><suffix> s <middle> p m` (SPM); the sample keeps its length (truncated or padded with the pad sentinel).
Cuts are made on the decoded text so they never split a token.  The random stream depends only on (seed, sample index).
Parity: `fast_llm/data/dataset/gpt/fim.py:13-212`.
"""

import numpy as np
import torch

from fast_llm_b200.data.document import LanguageModelDocument

MAX_SEED = 2**32


class GPTFimDataset:
    def __init__(self, config, dataset, sampling, seed: int):
        if sampling.use_preference_spans:
            raise NotImplementedError("Fill-in-the-middle cannot be combined with preference spans")
        self._config, self._dataset, self._seed = config, dataset, seed
        self._tokenizer = config.tokenizer.get_tokenizer()
        if self._tokenizer.bod_id is None or self._tokenizer.eod_id is None:
            raise ValueError("Fill-in-the-middle needs a tokenizer with both beginning- and end-of-document tokens")
        vocab = self._tokenizer.vocab
        self._suffix_id, self._prefix_id, self._middle_id, self._pad_id = (
            vocab[token] for token in (config.suffix_token, config.prefix_token, config.middle_token, config.pad_token))
        self._split_id = vocab[config.split_sample] if config.split_sample is not None else None

    def __len__(self) -> int:
        return len(self._dataset)

    @property
    def name(self) -> str:
        return f"{self._dataset.name}_fim"

    def __getitem__(self, index: int) -> list[LanguageModelDocument]:
        out = []
        for document in self._dataset[index]:
            if document.loss_masking_spans or document.chosen_span or document.image_patches is not None:
                raise NotImplementedError("Fill-in-the-middle supports plain token documents only")
            rng = np.random.RandomState(seed=(self._seed + index) % MAX_SEED)
            out.append(LanguageModelDocument(tokens=torch.from_numpy(self._transform_sample(document.tokens.numpy(), rng))))
        return out

    # ---- sample -> documents -> fragments
    def _split_apply(self, tokens: np.ndarray, separator: int, fn) -> np.ndarray:
        """Apply `fn` to the runs between `separator` tokens, keeping the separators."""
        cuts = np.flatnonzero(tokens == separator)
        if len(cuts) == 0:
            return fn(tokens)
        pieces, start = [], 0
        for cut in cuts:
            if cut > start:
                pieces += [fn(tokens[start:cut]), np.array([separator], dtype=tokens.dtype)]
            start = cut + 1
        pieces.append(fn(tokens[start:]))
        return np.concatenate(pieces)

    def _transform_sample(self, sample: np.ndarray, rng) -> np.ndarray:
        length = len(sample)
        result = self._split_apply(sample, self._tokenizer.eod, lambda doc: self._transform_document(doc, rng))
        if len(result) > length:
            result = result[:length]
        elif len(result) < length:
            result = np.concatenate([result, np.full(length - len(result), self._pad_id)])
        return result.astype(sample.dtype)

    def _transform_document(self, tokens: np.ndarray, rng) -> np.ndarray:
        c = self._config
        if self._split_id is None or not (tokens == self._split_id).any():
            return self._permute(tokens, rng, c.rate)
        if not rng.binomial(1, c.rate):
            return tokens
        return self._split_apply(tokens, self._split_id, lambda fragment: self._permute(fragment, rng, c.fragment_rate))

    # ---- the permutation itself
    def _permute(self, tokens: np.ndarray, rng, rate: float) -> np.ndarray:
        c = self._config
        if not rng.binomial(1, rate):
            return tokens
        text = self._tokenizer.detokenize(tokens)
        if c.ignore_prefix is not None and text.startswith(c.ignore_prefix):
            return tokens
        if c.max_middle_len is None:
            lo, hi = sorted(rng.randint(low=0, high=len(text) + 1, size=2).tolist())
        else:
            middle_length = rng.randint(low=0, high=min(c.max_middle_len, len(text)) + 1)
            lo = rng.randint(low=0, high=len(text) - middle_length + 1)
            hi = lo + middle_length
        dtype = torch.from_numpy(np.zeros(0, dtype=tokens.dtype)).dtype
        prefix = self._tokenizer.tokenize(text[:lo], end=False, data_type=dtype).numpy()
        middle = self._tokenizer.tokenize(text[lo:hi], begin=False, end=False, data_type=dtype).numpy()
        suffix = self._tokenizer.tokenize(text[hi:], begin=False, data_type=dtype).numpy()
        if c.truncate_or_pad:
            excess = len(prefix) + len(middle) + len(suffix) + 3 - len(tokens)
            if excess > 0:
                if len(suffix) <= excess:
                    return tokens
                suffix = suffix[: len(suffix) - excess]
            elif excess < 0:
                suffix = np.concatenate([suffix, np.full(-excess, self._pad_id)])
        if rng.binomial(1, c.spm_rate):
            parts = [[self._prefix_id, self._suffix_id], suffix, [self._middle_id], prefix, middle]
        else:
            parts = [[self._prefix_id], prefix, [self._suffix_id], suffix, [self._middle_id], middle]
        return np.concatenate([np.asarray(p, dtype=tokens.dtype) for p in parts])
