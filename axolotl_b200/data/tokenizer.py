"""Tokenizer loading: AutoTokenizer + special/added token overrides + pad-token fallback + chat
template resolution (behaviour of src/axolotl/loaders/tokenizer.py:130-336 and
src/axolotl/utils/chat_templates/base.py)."""
from __future__ import annotations

import os

from ..utils.logging import get_logger

LOG = get_logger(__name__)

# Named chat templates live as Jinja files under data/templates/ (one per model family; the formats are the
# public conversation layouts of those models). Anything else comes from the tokenizer or `chat_template_jinja`.
_TEMPLATE_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "templates")


class _TemplateTable(dict):
    """name -> template text, read from the template directory on first use."""

    def _load(self):
        if not self and os.path.isdir(_TEMPLATE_DIR):
            for fn in sorted(os.listdir(_TEMPLATE_DIR)):
                if fn.endswith(".jinja"):
                    with open(os.path.join(_TEMPLATE_DIR, fn), encoding="utf-8") as fh:
                        dict.__setitem__(self, fn[:-6], fh.read().rstrip("\n"))

    def __contains__(self, k):
        self._load()
        return dict.__contains__(self, k)

    def __getitem__(self, k):
        self._load()
        return dict.__getitem__(self, k)

    def __iter__(self):
        self._load()
        return dict.__iter__(self)

    def keys(self):
        self._load()
        return dict.keys(self)


CHAT_TEMPLATES = _TemplateTable()


def get_chat_template(name: str | None, tokenizer=None, jinja: str | None = None) -> str | None:
    """`tokenizer_default`, `tokenizer_default_fallback_<name>`, `jinja`, or a named template."""
    if name is None or name == "tokenizer_default":
        t = getattr(tokenizer, "chat_template", None) if tokenizer is not None else None
        if t is None and name == "tokenizer_default":
            raise ValueError("`chat_template: tokenizer_default` but the tokenizer has no chat template")
        return t
    if name.startswith("tokenizer_default_fallback_"):
        t = getattr(tokenizer, "chat_template", None) if tokenizer is not None else None
        return t or get_chat_template(name[len("tokenizer_default_fallback_"):], tokenizer, jinja)
    if name == "jinja":
        if not jinja:
            raise ValueError("`chat_template: jinja` needs `chat_template_jinja`")
        return open(jinja).read() if os.path.exists(jinja) else jinja
    if name in CHAT_TEMPLATES:
        return CHAT_TEMPLATES[name]
    raise ValueError(f"unknown chat template '{name}' (have: {sorted(CHAT_TEMPLATES)})")


def load_tokenizer(cfg):
    from transformers import AutoTokenizer

    src = cfg.get("tokenizer_config") or cfg.get("base_model_config") or cfg.get("base_model")
    if not src:
        raise ValueError("no tokenizer source: set `tokenizer_config` or `base_model`")
    kw = {}
    if cfg.get("tokenizer_use_fast") is not None:
        kw["use_fast"] = cfg["tokenizer_use_fast"]
    if cfg.get("tokenizer_legacy") is not None:
        kw["legacy"] = cfg["tokenizer_legacy"]
    tok = AutoTokenizer.from_pretrained(src, trust_remote_code=bool(cfg.get("trust_remote_code")), **kw)
    st = cfg.get("special_tokens") or {}
    for k in ("bos_token", "eos_token", "pad_token", "unk_token"):
        if st.get(k):
            tok.add_special_tokens({k: st[k]})
    if st.get("additional_special_tokens"):
        tok.add_special_tokens({"additional_special_tokens": list(st["additional_special_tokens"])})
    if cfg.get("tokens"):
        tok.add_tokens(list(cfg["tokens"]))
    if tok.pad_token is None:
        # same fallback the reference applies for Llama-style tokenizers
        tok.pad_token = tok.eos_token if tok.eos_token is not None else tok.unk_token
        LOG.info("tokenizer has no pad token: using %r", tok.pad_token)
    if cfg.get("chat_template"):
        tpl = get_chat_template(cfg["chat_template"], tok, cfg.get("chat_template_jinja"))
        if tpl:
            tok.chat_template = tpl
    return tok
