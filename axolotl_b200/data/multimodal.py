"""Multimodal chat data path: message normalisation, per-family role masking and the batch collator.

A multimodal sample is a conversation whose messages carry content parts (text, image, audio ...). The HF
*processor* of the model family renders the conversation with its chat template and produces token ids plus the
media tensors (``pixel_values`` ...); this module decides what the loss sees:

* ``normalize_example``: ``conversations`` (from / value) or a custom field -> OpenAI ``messages`` with list
  content; a column image (``images`` / ``image``) is attached to the bare ``{"type": "image"}`` placeholder, or to
  the first user turn; optional resize (exact size, or aspect-preserving pad to a square).
* ``role_keep_mask``: one left-to-right scan over the rendered token ids. A family declares, per role, the token
  sequence that opens a turn and the one that closes it (table ``FAMILY_MARKERS``); the longest opening marker wins
  at a position; tokens of trainable roles are kept, the closing marker follows ``train_on_eos`` (turn / all / none /
  last); a closing marker that also opens the next turn (``[/INST]``) is handed back to the scan.
* pad tokens and the family's media placeholder tokens never carry loss.
* ``MultiModalChatCollator``: strategy -> ``processor.apply_chat_template(tokenize=True, return_dict=True)`` ->
  ``labels``.

Same behaviour as the reference's processing strategies and collator
(src/axolotl/processing_strategies.py:46-1540, src/axolotl/utils/collators/mm_chat.py:15-59,
src/axolotl/loaders/processor.py:17-92). The vision / audio encoders of these families are not part of this
package's model graphs; the data path is usable with any model object that accepts the processor's batch.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field

import torch

from ..utils.logging import get_logger

LOG = get_logger(__name__)
IGNORE = -100
EOS_MODES = ("turn", "all", "none", "last")


@dataclass
class RoleBoundary:
    role: str
    start_tokens: list
    end_tokens: list = field(default_factory=list)   # empty: the turn runs to the end of the sequence
    include_start: bool = False
    include_end: bool = True


# family -> (closing marker, [(role, opening marker)], media placeholder token names, tokenizer attributes that
# name further media token ids). "eos" as a closing marker means the tokenizer's eos id; a ("role", start, end,
# include_end) 4-tuple overrides the family's closing marker for that role.
FAMILY_MARKERS = {
    "qwen2_vl": ("<|im_end|>", [(r, f"<|im_start|>{r}\n") for r in ("system", "user", "assistant")],
                 ("<|image_pad|>", "<|video_pad|>"), ()),
    "qwen3_5": ("<|im_end|>", [(r, f"<|im_start|>{r}\n") for r in ("system", "user", "assistant")],
                ("<|image_pad|>", "<|video_pad|>"), ()),
    "gemma3": ("<end_of_turn>", [("assistant", "<start_of_turn>model\n"), ("user", "<start_of_turn>user\n")],
               ("<image_soft_token>", "<start_of_image>"), ("boi_token",)),
    "gemma3n": ("<end_of_turn>", [("assistant", "<start_of_turn>model\n"), ("user", "<start_of_turn>user\n")],
                ("<image_soft_token>", "<audio_soft_token>"),
                ("image_token_id", "audio_token_id", "boi_token_id", "eoi_token_id")),
    "gemma4": ("<turn|>", [("assistant", "<|turn>model\n"), ("user", "<|turn>user\n"), ("system", "<|turn>system\n")],
               ("<|image|>", "<|audio|>", "<|image>", "<image|>", "<|audio>", "<audio|>"), ()),
    "llama3_2_vision": ("<|eot_id|>", [(r, f"<|start_header_id|>{r}<|end_header_id|>\n\n")
                                        for r in ("system", "user", "assistant", "ipython", "tool")], ("<|image|>",), ()),
    "llama4": ("<|eot|>", [(r, f"<|header_start|>{r}<|header_end|>\n\n")
                           for r in ("system", "user", "assistant", "ipython", "tool")],
               ("<|image|>", "<|patch|>", "<|image_start|>", "<|image_end|>"), ()),
    "pixtral": ("eos", [("user", "[INST]", "[/INST]", False), ("assistant", "[/INST]")], ("[IMG]", "[IMG_BREAK]", "[IMG_END]"), ()),
    "mistral_v7_tekken": ("eos", [("system", "[SYSTEM_PROMPT]", "[/SYSTEM_PROMPT]", True), ("user", "[INST]", "[/INST]", False),
                                  ("assistant", "[/INST]")], ("[IMG]", "[IMG_BREAK]", "[IMG_END]"), ()),
    # families whose templates give no token-level role markers: only pad and media tokens are masked until the
    # user declares `role_boundaries`
    "smolvlm2": (None, [], ("<image>",), ()),
    "internvl": (None, [], ("<IMG_CONTEXT>", "<img>", "</img>"), ()),
    "glm4v": (None, [], ("<|image|>", "<|begin_of_image|>", "<|end_of_image|>", "<|video|>", "<|begin_of_video|>",
                         "<|end_of_video|>"), ()),
    "voxtral": (None, [], ("[AUDIO]",), ()),
    "mistral3": (None, [], ("[IMG]", "[IMG_BREAK]", "[IMG_END]"), ()),
}


def _encode(tokenizer, text):
    return list(tokenizer.encode(text, add_special_tokens=False))


def family_boundaries(family: str, tokenizer) -> list[RoleBoundary]:
    """Role boundaries of a known family, encoded with ``tokenizer``; [] when a marker does not tokenise."""
    spec = FAMILY_MARKERS.get(family)
    if spec is None:
        return []
    close, roles = spec[0], spec[1]
    if not roles:
        return []

    def closing(marker):
        if marker == "eos":
            eos = getattr(tokenizer, "eos_token_id", None)
            return [eos] if eos is not None else []
        return _encode(tokenizer, marker)

    default_end = closing(close)
    out = []
    for entry in roles:
        role, start = entry[0], _encode(tokenizer, entry[1])
        end, include_end = (closing(entry[2]), entry[3]) if len(entry) == 4 else (default_end, True)
        if start and end:
            out.append(RoleBoundary(role, start, end, include_end=include_end))
    return out


def resolve_role_boundaries(specs, tokenizer) -> list[RoleBoundary]:
    """User-declared boundaries (``role_boundaries:`` in the YAML): ``{role, start, end?, include_start?,
    include_end?}``; ``end: eos_token`` is the tokenizer's eos id, a missing ``end`` runs to the end of the row."""
    out = []
    for i, spec in enumerate(specs):
        d = dict(spec) if isinstance(spec, dict) else (spec.model_dump() if callable(getattr(spec, "model_dump", None)) else dict(spec))
        if not d.get("role") or d.get("start") is None:
            raise ValueError(f"role_boundaries[{i}] needs both 'role' and 'start' (got {d!r})")
        start = _encode(tokenizer, d["start"])
        if not start:
            raise ValueError(f"role_boundaries[{i}]: start marker {d['start']!r} tokenises to nothing")
        end_spec = d.get("end")
        if end_spec is None:
            end = []
        elif end_spec == "eos_token":
            if getattr(tokenizer, "eos_token_id", None) is None:
                raise ValueError(f"role_boundaries[{i}] asks for end='eos_token' but the tokenizer has no eos token")
            end = [tokenizer.eos_token_id]
        else:
            end = _encode(tokenizer, end_spec)
            if not end:
                raise ValueError(f"role_boundaries[{i}]: end marker {end_spec!r} tokenises to nothing "
                                 f"(use end: null or end: eos_token)")
        out.append(RoleBoundary(d["role"], start, end, bool(d.get("include_start", False)), bool(d.get("include_end", True))))
    return out


def role_keep_mask(rows, boundaries, roles_to_train=("assistant",), train_on_eos="turn") -> torch.Tensor:
    """[B, L] bool: True where a token contributes to the loss. ``rows``: [B, L] tensor or list of id lists."""
    if train_on_eos not in EOS_MODES:
        raise ValueError(f"train_on_eos={train_on_eos!r} is not one of {EOS_MODES}")
    rows = rows.tolist() if torch.is_tensor(rows) else [list(r) for r in rows]
    train = set(roles_to_train)
    # opening markers indexed by their first token, longest first, so a position is settled by one dict lookup
    by_first = {}
    for b in boundaries:
        if b.start_tokens:
            by_first.setdefault(b.start_tokens[0], []).append(b)
    for lst in by_first.values():
        lst.sort(key=lambda b: -len(b.start_tokens))
    keep = torch.zeros((len(rows), max((len(r) for r in rows), default=0)), dtype=torch.bool)
    for i, ids in enumerate(rows):
        n, j, last_end = len(ids), 0, None
        while j < n:
            hit = None
            for b in by_first.get(ids[j], ()):
                m = len(b.start_tokens)
                if ids[j:j + m] == b.start_tokens:
                    hit = b
                    break
            if hit is None:
                j += 1
                continue
            body = j + len(hit.start_tokens)
            m = len(hit.end_tokens)
            stop, found = n, False
            if m:
                first = hit.end_tokens[0]
                q = body
                while q + m <= n:
                    if ids[q] == first and ids[q:q + m] == hit.end_tokens:
                        stop, found = q, True
                        break
                    q += 1
            after = stop + m if found else n
            if hit.role in train:
                if hit.include_start:
                    keep[i, j:body] = True
                keep[i, body:stop] = True
                if found and hit.include_end:
                    if train_on_eos in ("turn", "all"):
                        keep[i, stop:after] = True
                    elif train_on_eos == "last":
                        last_end = (stop, after)
            elif found and hit.include_end and train_on_eos == "all":
                keep[i, stop:after] = True
            # a closing marker that is not part of the turn may open the next one: scan it again
            j = stop if (found and not hit.include_end) else after
        if last_end is not None:
            keep[i, last_end[0]:last_end[1]] = True
    return keep


def _load_image(value):
    """PIL image from a PIL image, path, URL-less bytes or base64 string (PIL is optional: values pass through
    untouched without it)."""
    try:
        from PIL import Image
    except ImportError:
        return value
    if isinstance(value, Image.Image):
        return value
    if isinstance(value, (bytes, bytearray)):
        import io

        return Image.open(io.BytesIO(value)).convert("RGB")
    if isinstance(value, dict) and value.get("bytes"):
        import io

        return Image.open(io.BytesIO(value["bytes"])).convert("RGB")
    if isinstance(value, dict) and value.get("path"):
        value = value["path"]
    if isinstance(value, str):
        import os

        if os.path.exists(value):
            return Image.open(value).convert("RGB")
        if value.startswith("data:image"):
            import base64
            import io

            return Image.open(io.BytesIO(base64.b64decode(value.split(",", 1)[1]))).convert("RGB")
    return value


def _resize(img, size, algorithm=None):
    if size is None or not hasattr(img, "resize"):
        return img
    from PIL import Image, ImageOps

    algo = algorithm if algorithm is not None else Image.Resampling.BILINEAR
    if isinstance(size, (tuple, list)):
        return img.resize(tuple(size), algo)
    return ImageOps.pad(img, (int(size), int(size)), method=algo, color=(0, 0, 0))   # keep the aspect, pad to a square


def _drop_none(x):
    if isinstance(x, dict):
        return {k: _drop_none(v) for k, v in x.items() if v is not None}
    if isinstance(x, list):
        return [_drop_none(v) for v in x]
    return x


_ROLE_ALIASES = {"human": "user", "gpt": "assistant"}


def normalize_example(example: dict, field_messages=("messages",), image_size=None, resize_algorithm=None) -> dict:
    """One dataset row -> ``{"messages": [{"role", "content": [parts]}], ...}`` with its column image attached."""
    names = (field_messages,) if isinstance(field_messages, str) else tuple(n for n in (field_messages or ("messages",)) if n)
    src = next((n for n in names if example.get(n) is not None), None)
    if src is None and example.get("messages") is not None:
        src = "messages"
    ex = copy.deepcopy(example)
    msgs = None
    if src is not None:
        msgs = ex.pop(src)
    elif "conversations" in ex:
        msgs = ex.pop("conversations")
    elif "messages" in ex:
        raise ValueError("`messages` is present but None; provide non-null `messages` or a `conversations` field")
    else:
        raise ValueError("only the configured `field_messages`, `messages` and `conversations` hold conversations")
    if msgs and isinstance(msgs[0], dict) and "from" in msgs[0] and "value" in msgs[0]:      # ShareGPT schema
        msgs = [{"role": _ROLE_ALIASES.get(m["from"], m["from"]), "content": m["value"]} for m in msgs]
    ex.pop("conversations", None)
    out = []
    for m in msgs:
        c = m["content"]
        if isinstance(c, str):
            c = [{"type": "text", "text": c}]
        out.append({"role": m["role"], "content": c})
    ex["messages"] = out
    key = next((k for k in ("images", "image") if ex.get(k) is not None), None)
    if key is not None:
        vals = ex[key] if isinstance(ex[key], (list, tuple)) else [ex[key]]
        if len(vals) > 1:
            LOG.warning("a sample carries %d column images; the first one is used (put several images into "
                        "multi-content messages instead)", len(vals))
        img = _resize(_load_image(vals[0]), image_size, resize_algorithm)
        slot = None
        for m in out:
            for part in m["content"]:
                if part.get("type") == "image" and not any(k in part for k in ("image", "url", "path", "base64")):
                    slot = part
                    break
            if slot is not None:
                break
        if slot is not None:
            slot["image"] = img
        else:
            first_user = next((m for m in out if m["role"] == "user"), out[0])
            first_user["content"].append({"type": "image", "image": img})
    return _drop_none(ex)


class ProcessingStrategy:
    """What one model family's processor needs around it: normalised messages in, masked labels out."""

    def __init__(self, processor, family=None, chat_template=None, image_size=None, image_resize_algorithm=None,
                 train_on_inputs=False, roles_to_train=None, train_on_eos=None, role_boundaries=None, field_messages=None):
        self.processor = processor
        self.tokenizer = getattr(processor, "tokenizer", processor)
        self.family = family
        self.chat_template = chat_template
        self.image_size, self.image_resize_algorithm = image_size, image_resize_algorithm
        self.train_on_inputs = bool(train_on_inputs)
        self.roles_to_train = list(roles_to_train) if roles_to_train is not None else ["assistant"]
        self.train_on_eos = train_on_eos if train_on_eos is not None else "turn"
        if self.train_on_eos not in EOS_MODES:
            raise ValueError(f"train_on_eos={self.train_on_eos!r} is not one of {EOS_MODES}")
        self.field_messages = field_messages
        built_in = family_boundaries(family, self.tokenizer) if family else []
        self.boundaries = resolve_role_boundaries(role_boundaries, self.tokenizer) if role_boundaries else built_in
        self.media_ids = self._media_token_ids()
        self._warned = False
        LOG.info("multimodal strategy: family=%s train_on_inputs=%s roles_to_train=%s train_on_eos=%s boundaries=%d (%s)",
                 family, self.train_on_inputs, self.roles_to_train, self.train_on_eos, len(self.boundaries),
                 "override" if role_boundaries else "built-in")

    def _media_token_ids(self):
        tok, ids = self.tokenizer, set()
        unk = getattr(tok, "unk_token_id", None)
        image_token = getattr(self.processor, "image_token", None)
        names = list(FAMILY_MARKERS.get(self.family, (None, None, (), ()))[2]) + ([image_token] if image_token else [])
        for name in names:
            try:
                i = tok.convert_tokens_to_ids(name)
            except Exception:   # noqa: BLE001 - tokenizers differ in how they refuse unknown tokens
                i = None
            if isinstance(i, int) and i >= 0 and i != unk:
                ids.add(i)
        for attr in FAMILY_MARKERS.get(self.family, (None, None, (), ()))[3]:
            v = getattr(tok, attr, None)
            if isinstance(v, str):
                v = tok.convert_tokens_to_ids(v)
            if isinstance(v, int) and v != unk:
                ids.add(v)
        for attr in ("image_token_id", "video_token_id", "audio_token_id"):
            v = getattr(self.processor, attr, None)
            if isinstance(v, int):
                ids.add(v)
        for v in getattr(self.processor, "image_ids", None) or ():     # InternVL: several image token ids
            if isinstance(v, int):
                ids.add(v)
        if self.family == "gemma3" and not any(True for _ in ids):
            ids.add(262144)      # the soft image token of the released tokenizer
        return sorted(ids)

    def __call__(self, examples):
        return [normalize_example(e, self.field_messages or ("messages",), self.image_size, self.image_resize_algorithm)
                for e in examples]

    def keep_mask(self, input_ids):
        if self.train_on_inputs:
            return torch.ones_like(input_ids, dtype=torch.bool)
        if not self.boundaries:
            if not self._warned:
                self._warned = True
                LOG.warning("no role boundaries are known for family %r: train_on_inputs / roles_to_train / train_on_eos "
                            "cannot restrict the loss, only pad and media tokens are masked. Declare `role_boundaries` "
                            "in the config to enable assistant-only training.", self.family)
            return torch.ones_like(input_ids, dtype=torch.bool)
        return role_keep_mask(input_ids, self.boundaries, self.roles_to_train, self.train_on_eos).to(input_ids.device)

    def process_labels(self, input_ids):
        keep = self.keep_mask(input_ids)
        pad = getattr(self.tokenizer, "pad_token_id", None)
        if pad is not None:
            keep = keep & (input_ids != pad)
        for i in self.media_ids:
            keep = keep & (input_ids != i)
        labels = input_ids.clone()
        labels[~keep] = IGNORE
        return labels


_PROCESSOR_CLASS_FAMILY = {"Qwen2VLProcessor": "qwen2_vl", "Qwen2_5_VLProcessor": "qwen2_vl", "Qwen3VLProcessor": "qwen2_vl",
                           "Gemma3Processor": "gemma3", "Gemma3nProcessor": "gemma3n", "MllamaProcessor": "llama3_2_vision",
                           "Llama4Processor": "llama4", "PixtralProcessor": "pixtral", "VoxtralProcessor": "voxtral",
                           "SmolVLMProcessor": "smolvlm2", "InternVLProcessor": "internvl", "Glm4vProcessor": "glm4v",
                           "Glm46VProcessor": "glm4v", "Mistral3Processor": "mistral3"}


def get_processing_strategy(processor, chat_template=None, chat_template_type=None, **kw) -> ProcessingStrategy:
    """The strategy for ``chat_template_type`` (a family name), else for the processor's class, else the generic one
    (pad / media masking only until ``role_boundaries`` are declared)."""
    family = chat_template_type if chat_template_type in FAMILY_MARKERS else _PROCESSOR_CLASS_FAMILY.get(type(processor).__name__)
    if chat_template is None and chat_template_type in (None, "tokenizer_default"):
        chat_template = getattr(getattr(processor, "tokenizer", processor), "chat_template", None)
    return ProcessingStrategy(processor, family=family, chat_template=chat_template, **kw)


def load_processor(cfg, tokenizer=None):
    """``AutoProcessor`` for ``processor_config`` / ``base_model`` (``processor_type`` picks a class by name); the
    already-configured tokenizer (added tokens, pad token, chat template) replaces the processor's own."""
    import transformers

    src = cfg.get("processor_config") or cfg.get("base_model_config") or cfg.get("base_model")
    cls = getattr(transformers, cfg["processor_type"]) if cfg.get("processor_type") else transformers.AutoProcessor
    kw = {"trust_remote_code": bool(cfg.get("trust_remote_code"))}
    if cfg.get("revision_of_model"):
        kw["revision"] = cfg["revision_of_model"]
    processor = cls.from_pretrained(src, **kw)
    if tokenizer is not None and hasattr(processor, "tokenizer"):
        processor.tokenizer = tokenizer
    size = cfg.get("image_size")
    ip = getattr(processor, "image_processor", None)
    if size and ip is not None and hasattr(ip, "size"):        # keep the processor's own resize in step with ours
        if isinstance(size, (tuple, list)):
            ip.size = {"height": int(size[1]), "width": int(size[0])}
        else:
            ip.size = {"height": int(size), "width": int(size)}
    return processor


class MultiModalChatCollator:
    """Rows of conversations -> one padded batch from the family's processor, with ``labels``. Sample packing is
    refused: media tensors are tied to their own row."""

    def __init__(self, tokenizer, processing_strategy: ProcessingStrategy, packing=False, padding=True):
        if packing:
            raise ValueError("sample packing is not available for multimodal batches")
        self.tokenizer, self.strategy, self.padding = tokenizer, processing_strategy, padding

    def __call__(self, examples):
        rows = self.strategy(examples)
        batch = self.strategy.processor.apply_chat_template(
            [r["messages"] for r in rows], add_generation_prompt=False, tokenize=True, return_tensors="pt",
            return_dict=True, chat_template=self.strategy.chat_template, processor_kwargs={"padding": self.padding})
        batch["labels"] = self.strategy.process_labels(batch["input_ids"])
        return batch


MEDIA_TENSOR_KEYS = ("pixel_values",)


def unpad_batch(batch, pad_token_id=None) -> dict:
    """The processor's padded [B, S] batch -> one padding-free row for the varlen kernels: the real tokens of every
    conversation back to back with positions restarting at each, the media tensors alongside (row order kept, so image i
    still meets its placeholder tokens)."""
    ids, labels = batch["input_ids"], batch["labels"]
    mask = batch.get("attention_mask")
    if mask is None:
        mask = torch.ones_like(ids) if pad_token_id is None else (ids != pad_token_id).long()
    keep = mask.bool()
    lens = keep.sum(1)
    pos = (keep.long().cumsum(1) - 1).clamp(min=0)
    out = {"input_ids": ids[keep][None].contiguous(), "labels": labels[keep][None].contiguous(),
           "position_ids": pos[keep][None].to(torch.int32).contiguous(),
           "cu_seqlens": torch.cat([torch.zeros(1, dtype=torch.int32), lens.cumsum(0).to(torch.int32)]),
           "aux_tensors": {k: batch[k] for k in MEDIA_TENSOR_KEYS if batch.get(k) is not None}}
    return out


class RawConversationDataset:
    """Untokenised multimodal rows: the processor renders and tokenises them batch by batch (media tensors are too large
    to prepare ahead)."""

    def __init__(self, rows):
        self.rows = rows
        self.lengths = None

    def __len__(self):
        return len(self.rows)

    def __getitem__(self, i):
        return self.rows[int(i)]


def make_multimodal_batches_fn(cfg, ds, collator, rank, dp_size, is_eval=False):
    """callable(epoch) -> iterator of padding-free micro-batches of ``micro_batch_size`` conversations for this rank."""
    import numpy as np

    mbs = (cfg.get("eval_batch_size") if is_eval else cfg.get("micro_batch_size")) or 1
    seq = cfg.get("sequence_len")
    pad = getattr(collator.tokenizer, "pad_token_id", None)

    def batches(epoch=0):
        n = len(ds)
        order = np.arange(n) if is_eval else np.random.default_rng((cfg.get("seed") or 42) + epoch).permutation(n)
        mine = order[rank::dp_size]
        if not is_eval:
            mine = mine[: (n // (mbs * dp_size)) * mbs]
        for i in range(0, len(mine), mbs):
            idx = mine[i:i + mbs]
            if len(idx) < mbs and not is_eval:
                break
            b = collator([ds[j] for j in idx])
            if seq and b["input_ids"].shape[1] > seq:
                raise ValueError(f"a multimodal conversation renders to {b['input_ids'].shape[1]} tokens, sequence_len is {seq}: "
                                 "truncation would cut through image placeholder tokens; raise sequence_len or drop the row")
            yield unpad_batch(b, pad)

    return batches
