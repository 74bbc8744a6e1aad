"""Documents, packed batches and per-micro-sequence model inputs.

A micro-batch is a flat stream of `micro_batch_size` tokens packed from one or more documents (plus the extra tokens
needed as labels).  `LanguageModelBatch.get_model_inputs` turns it into one `LanguageModelInput` per micro-sequence:
the token slice of this sequence-data-parallel rank, labels for each prediction distance (masked across document
boundaries, by loss-masking spans and on padding), document boundaries as `cu_seqlens` for variable-length attention,
positions, document indices and label counts.  Parity: `fast_llm/data/document/language_model.py:107-238`,
`fast_llm/data/document/block.py:64-178`.
"""

import dataclasses

import torch

from fast_llm_b200.layers.kwargs import BlockKwargs, LanguageModelKwargs


@dataclasses.dataclass
class LanguageModelDocument:
    tokens: torch.Tensor
    loss_masking_spans: list[tuple[int, int]] | None = None
    chosen_span: tuple[int, int] | None = None
    rejected_span: tuple[int, int] | None = None
    image_patches: torch.Tensor | None = None  # [num_patches, channels, height, width]
    image_patch_positions: torch.Tensor | None = None  # token position of every patch
    image_patch_coordinates: torch.Tensor | None = None  # [num_patches, 2] (row, column) inside its image
    advantages: torch.Tensor | None = None
    old_log_probabilities: torch.Tensor | None = None

    def __len__(self) -> int:
        return len(self.tokens)

    def crop(self, begin: int, end: int) -> "LanguageModelDocument":
        def crop_spans(spans):
            if spans is None:
                return None
            out = [(max(b, begin) - begin, min(e, end) - begin) for b, e in spans if e > begin and b < end]
            return out

        def crop_span(span):
            got = crop_spans([span]) if span is not None else None
            return got[0] if got else None

        patches = positions = coordinates = None
        if self.image_patches is not None:
            keep = (self.image_patch_positions >= begin) & (self.image_patch_positions < end)
            patches, positions = self.image_patches[keep], self.image_patch_positions[keep] - begin
            coordinates = None if self.image_patch_coordinates is None else self.image_patch_coordinates[keep]
        return LanguageModelDocument(
            tokens=self.tokens[begin:end], loss_masking_spans=crop_spans(self.loss_masking_spans),
            chosen_span=crop_span(self.chosen_span), rejected_span=crop_span(self.rejected_span),
            image_patches=patches, image_patch_positions=positions, image_patch_coordinates=coordinates,
            advantages=None if self.advantages is None else self.advantages[begin:end],
            old_log_probabilities=None if self.old_log_probabilities is None else self.old_log_probabilities[begin:end])


@dataclasses.dataclass
class LanguageModelInput:
    """One micro-sequence on one rank, still on the host (pinned when a GPU will consume it)."""

    tokens: torch.Tensor  # [tokens_local]
    labels: dict[int, torch.Tensor]  # prediction distance -> [tokens_local], -100 = ignore
    position_ids: torch.Tensor  # int32 [tokens_local]
    document_index: torch.Tensor  # int32 [tokens_local]
    cu_seqlens_q: torch.Tensor  # int32
    cu_seqlens_k: torch.Tensor  # int32
    max_seqlen_q: int
    max_seqlen_k: int
    num_tokens: int  # tokens of the whole micro-sequence (all sequence-data ranks)
    num_labels: dict[int, int]  # valid labels of the whole micro-BATCH per prediction distance
    sequence_k_end: int  # number of keys (prefix + this rank's part) this rank's queries may see
    micro_sequence_index: int = 0
    extras: dict = dataclasses.field(default_factory=dict)

    def pin_memory(self):
        for f in ("tokens", "position_ids", "document_index", "cu_seqlens_q", "cu_seqlens_k"):
            setattr(self, f, getattr(self, f).pin_memory())
        self.labels = {d: t.pin_memory() for d, t in self.labels.items()}
        self.extras = {k: (v.pin_memory() if torch.is_tensor(v) else v) for k, v in self.extras.items()}
        return self

    def nbytes(self) -> int:
        tensors = [self.tokens, self.position_ids, self.document_index, self.cu_seqlens_q, self.cu_seqlens_k,
                   *self.labels.values(), *(v for v in self.extras.values() if torch.is_tensor(v))]
        return sum(t.numel() * t.element_size() for t in tensors)

    def to_kwargs(self, device) -> dict:
        move = lambda t: t.to(device, non_blocking=True)
        kwargs = {
            LanguageModelKwargs.token_ids: move(self.tokens),
            LanguageModelKwargs.position_ids: move(self.position_ids),
            LanguageModelKwargs.document_index: move(self.document_index),
            LanguageModelKwargs.cu_seqlens_q: move(self.cu_seqlens_q),
            LanguageModelKwargs.cu_seqlens_k: move(self.cu_seqlens_k),
            LanguageModelKwargs.max_seqlen_q: self.max_seqlen_q,
            LanguageModelKwargs.max_seqlen_k: self.max_seqlen_k,
            LanguageModelKwargs.num_tokens: self.num_tokens,
            LanguageModelKwargs.micro_sequence_index: self.micro_sequence_index,
            LanguageModelKwargs.sequence_k_offset: self.sequence_k_end,
            "max_position": int(self.extras.get("max_position", self.max_seqlen_k)),
        }
        for distance, labels in self.labels.items():
            key = LanguageModelKwargs.labels if distance == 1 else f"{LanguageModelKwargs.labels}_{distance}"
            kwargs[key] = move(labels)
            count = torch.tensor([1.0 / max(self.num_labels[distance], 1)], dtype=torch.float32)
            kwargs[f"_inverse_label_count_{distance}"] = move(count)
        for key, value in self.extras.items():
            if key != "max_position":
                kwargs[key] = move(value) if torch.is_tensor(value) else value
        return kwargs


@dataclasses.dataclass
class LanguageModelBatch:
    """A packed micro-batch: `tokens` holds micro_batch_size + predicted_tokens entries (padded with -100)."""

    tokens: torch.Tensor
    document_lengths: list[int]
    loss_mask: torch.Tensor | None = None  # bool [len(tokens)], False = never a label
    chosen_spans: list[tuple[int, int]] | None = None
    rejected_spans: list[tuple[int, int]] | None = None
    advantages: torch.Tensor | None = None
    old_log_probabilities: torch.Tensor | None = None
    image_patches: torch.Tensor | None = None
    image_patch_positions: torch.Tensor | None = None
    image_patch_coordinates: torch.Tensor | None = None

    @classmethod
    def from_documents(cls, documents: list[LanguageModelDocument], size: int, use_loss_masking_spans: bool = True) -> "LanguageModelBatch":
        tokens = torch.full((size,), -100, dtype=torch.int64)
        loss_mask = None
        chosen, rejected = [], []
        lengths = []
        advantages = old = None
        patches, patch_pos, patch_coord = [], [], []
        offset = 0
        for doc in documents:
            n = min(len(doc), size - offset)
            if n <= 0:
                break
            tokens[offset : offset + n] = doc.tokens[:n].to(torch.int64)
            if use_loss_masking_spans and doc.loss_masking_spans:
                if loss_mask is None:
                    loss_mask = torch.ones(size, dtype=torch.bool)
                for b, e in doc.loss_masking_spans:
                    loss_mask[offset + b : offset + min(e, n)] = False
            if doc.chosen_span is not None:
                chosen.append((offset + doc.chosen_span[0], offset + min(doc.chosen_span[1], n)))
            if doc.rejected_span is not None:
                rejected.append((offset + doc.rejected_span[0], offset + min(doc.rejected_span[1], n)))
            if doc.advantages is not None:
                if advantages is None:
                    advantages = torch.zeros(size, dtype=torch.float32)
                    old = torch.zeros(size, dtype=torch.float32)
                advantages[offset : offset + n] = doc.advantages[:n]
                if doc.old_log_probabilities is not None:
                    old[offset : offset + n] = doc.old_log_probabilities[:n]
            if doc.image_patches is not None and len(doc.image_patches):
                keep = doc.image_patch_positions < n
                patches.append(doc.image_patches[keep])
                patch_pos.append(doc.image_patch_positions[keep] + offset)
                if doc.image_patch_coordinates is not None:
                    patch_coord.append(doc.image_patch_coordinates[keep])
            lengths.append(n)
            offset += n
        if offset < size:
            lengths.append(size - offset)  # padding behaves as one more document, all labels ignored
        return cls(tokens=tokens, document_lengths=lengths, loss_mask=loss_mask, chosen_spans=chosen or None,
                   rejected_spans=rejected or None, advantages=advantages, old_log_probabilities=old,
                   image_patches=torch.cat(patches) if patches else None,
                   image_patch_positions=torch.cat(patch_pos) if patch_pos else None,
                   image_patch_coordinates=torch.cat(patch_coord) if patch_coord else None)

    def get_model_inputs(self, *, micro_batch_size: int, predicted_tokens: int = 1, micro_batch_splits: int = 1,
                         sequence_data_parallel: int = 1, sequence_data_rank: int = 0, causal: bool = True,
                         cross_document_attention: bool = False, pin: bool = False) -> list[LanguageModelInput]:
        size = micro_batch_size
        tokens = self.tokens
        assert len(tokens) >= size + predicted_tokens, (len(tokens), size, predicted_tokens)
        lengths = list(self.document_lengths)
        # document id and in-document position of every token of the extended sequence
        doc_index = torch.repeat_interleave(torch.arange(len(lengths)), torch.tensor(lengths))[: len(tokens)]
        starts = torch.cumsum(torch.tensor([0] + lengths[:-1]), 0)
        positions = torch.arange(len(tokens)) - starts[doc_index]
        if cross_document_attention:
            doc_index = torch.zeros_like(doc_index)
            positions = torch.arange(len(tokens))
            lengths = [len(tokens)]
            starts = torch.tensor([0])
        inputs_tokens = tokens[:size]  # negative ids (image placeholders, padding) stay: the embedding layer maps them to zero
        labels, num_labels = {}, {}
        for d in range(1, predicted_tokens + 1):
            lab = tokens[d : d + size].clone()
            same_doc = doc_index[d : d + size] == doc_index[:size]
            lab[~same_doc] = -100
            if self.loss_mask is not None:
                lab[~self.loss_mask[d : d + size]] = -100
            lab[tokens[:size] < 0] = -100
            labels[d] = lab
            num_labels[d] = int((lab >= 0).sum())
        doc_ends = (starts + torch.tensor(lengths)).tolist()
        doc_starts = starts.tolist()
        chunk = size // micro_batch_splits
        assert chunk * micro_batch_splits == size
        part = chunk // sequence_data_parallel
        assert part * sequence_data_parallel == chunk
        out = []
        for m in range(micro_batch_splits):
            q_begin = m * chunk + sequence_data_rank * part
            q_end = q_begin + part
            k_end = q_end  # keys: everything up to the end of this rank's queries
            cu_q, cu_k = [0], [0]
            max_q = max_k = 0
            for s, e in zip(doc_starts, doc_ends):
                if s >= k_end:
                    break
                kb, ke = s, min(e, k_end)
                qb, qe = max(s, q_begin), min(e, q_end)
                qlen = max(qe - qb, 0)
                cu_q.append(cu_q[-1] + qlen)
                cu_k.append(cu_k[-1] + (ke - kb))
                max_q, max_k = max(max_q, qlen), max(max_k, ke - kb)
            sl = slice(q_begin, q_end)
            extras = {"max_position": int(positions[:size].max()) if size else 0}
            if bool((inputs_tokens[sl] < 0).any()):
                extras[LanguageModelKwargs.mask_inputs] = True
            if self.advantages is not None:
                extras[LanguageModelKwargs.advantages] = self.advantages[1 : size + 1][sl].clone()
                extras[LanguageModelKwargs.old_log_probabilities] = self.old_log_probabilities[1 : size + 1][sl].clone()
            if self.chosen_spans is not None and m == 0:
                # spans are given in label coordinates (position of the predicted token - 1)
                extras[LanguageModelKwargs.chosen_spans] = [(max(b - 1, 0), max(e - 1, 0)) for b, e in self.chosen_spans]
                extras[LanguageModelKwargs.rejected_spans] = [(max(b - 1, 0), max(e - 1, 0)) for b, e in (self.rejected_spans or [])]
            if self.image_patches is not None and m == 0:
                extras["image_patches"] = self.image_patches
                extras["image_patch_positions"] = self.image_patch_positions
                if self.image_patch_coordinates is not None:
                    extras["patch_positions"] = self.image_patch_coordinates
            inp = LanguageModelInput(
                tokens=inputs_tokens[sl].clone(), labels={d: lab[sl].clone() for d, lab in labels.items()},
                position_ids=positions[:size][sl].to(torch.int32), document_index=doc_index[:size][sl].to(torch.int32),
                cu_seqlens_q=torch.tensor(cu_q, dtype=torch.int32), cu_seqlens_k=torch.tensor(cu_k, dtype=torch.int32),
                max_seqlen_q=max_q, max_seqlen_k=max_k, num_tokens=chunk, num_labels=num_labels, sequence_k_end=k_end,
                micro_sequence_index=m, extras=extras)
            out.append(inp.pin_memory() if pin else inp)
        return out
