"""Prompt strategies: raw dataset rows -> {input_ids, labels, attention_mask}.

Label masking rules follow the reference (src/axolotl/prompt_tokenizers.py:43-381,
src/axolotl/prompt_strategies/chat_template.py:278-1086):
* instruction formats: prompt tokens are -100 unless ``train_on_inputs``; the response is
  tokenised separately with BOS stripped and EOS appended; everything is truncated to
  ``sequence_len``.
* chat templates: all labels start at -100; a turn is trainable when its role is in
  ``roles_to_train`` (default assistant) or its ``training`` field says so; the token span of a
  turn is found by rendering the conversation up to and including that turn; EOS/EOT handling via
  ``train_on_eos`` / ``train_on_eot`` in {all, turn, last}.
"""
from __future__ import annotations

import numpy as np

IGNORE_INDEX = -100

ALPACA_SYSTEM_INPUT = ("Below is an instruction that describes a task, paired with an input that provides further "
                       "context. Write a response that appropriately completes the request.\n\n")
ALPACA_SYSTEM_NO_INPUT = ("Below is an instruction that describes a task. Write a response that appropriately "
                          "completes the request.\n\n")


def _tok(tokenizer, text, add_bos=True, add_eos=False, max_len=None):
    ids = tokenizer(text, add_special_tokens=False)["input_ids"]
    if add_bos and tokenizer.bos_token_id is not None:
        ids = [tokenizer.bos_token_id] + ids
    if add_eos and tokenizer.eos_token_id is not None and (not ids or ids[-1] != tokenizer.eos_token_id):
        ids = ids + [tokenizer.eos_token_id]
    if max_len is not None:
        ids = ids[:max_len]
    return ids


def _pack(ids, labels):
    return {"input_ids": list(ids), "labels": list(labels), "attention_mask": [1] * len(ids)}


class Strategy:
    """Base: ``tokenize(row) -> dict`` (or None to drop the row)."""

    def __init__(self, tokenizer, cfg, ds_cfg=None):
        self.tok, self.cfg, self.ds_cfg = tokenizer, cfg, ds_cfg or {}
        self.seq_len = cfg.get("sequence_len") or 2048
        self.train_on_inputs = bool(cfg.get("train_on_inputs"))

    def prompt_response(self, row):
        raise NotImplementedError

    def tokenize(self, row):
        prompt, response = self.prompt_response(row)
        p = _tok(self.tok, prompt, add_bos=True, add_eos=False, max_len=self.seq_len)
        r = _tok(self.tok, response, add_bos=False, add_eos=True, max_len=max(self.seq_len - len(p), 0))
        ids = p + r
        labels = (p if self.train_on_inputs else [IGNORE_INDEX] * len(p)) + r
        return _pack(ids, labels)


class AlpacaStrategy(Strategy):
    style = "instruct"  # "instruct" | "chat"

    def fields(self, row):
        return row.get("instruction", ""), row.get("input", ""), row.get("output", "")

    def prompt_response(self, row):
        ins, inp, out = self.fields(row)
        if self.style == "chat":
            turn = "USER: {} ASSISTANT:"
            body = f"{ins}\n{inp}" if inp else ins
            sys_ = ALPACA_SYSTEM_INPUT if inp else ALPACA_SYSTEM_NO_INPUT
            return sys_ + turn.format(body), " " + out if out else out
        if inp:
            return f"{ALPACA_SYSTEM_INPUT}### Instruction:\n{ins}\n\n### Input:\n{inp}\n\n### Response:\n", out
        return f"{ALPACA_SYSTEM_NO_INPUT}### Instruction:\n{ins}\n\n### Response:\n", out


class AlpacaChatStrategy(AlpacaStrategy):
    style = "chat"


class GPTeacherStrategy(AlpacaStrategy):
    def fields(self, row):
        return row.get("instruction", ""), row.get("input", ""), row.get("response", "")


class OpenAssistantStrategy(AlpacaStrategy):
    def fields(self, row):
        return row.get("INSTRUCTION", ""), "", row.get("RESPONSE", "")


class JeopardyStrategy(AlpacaStrategy):
    def fields(self, row):
        return row.get("question", ""), row.get("category", ""), "what is " + str(row.get("answer", ""))


class SummarizeTLDRStrategy(AlpacaStrategy):
    def fields(self, row):
        return "Summarize the following article as a TL;DR.", row.get("article", ""), row.get("summary", "")


class UserDefinedStrategy(Strategy):
    """``type:`` given as a dict with field names and format strings."""

    def prompt_response(self, row):
        t = self.ds_cfg.get("type") if isinstance(self.ds_cfg.get("type"), dict) else {}
        ins = row.get(t.get("field_instruction") or "instruction", "")
        inp = row.get(t.get("field_input") or "input", "")
        out = row.get(t.get("field_output") or "output", "")
        system = row.get(t.get("field_system") or "system", "") or t.get("system_prompt") or ""
        fmt = (t.get("format") if inp else (t.get("no_input_format") or t.get("format"))) or "{instruction} {input} "
        sysfmt = t.get("system_format") or "{system}"
        prompt = (sysfmt.format(system=system) if system else "") + fmt.format(instruction=ins, input=inp)
        return prompt, out


class CompletionStrategy(Strategy):
    """Raw text; every token is trained (optionally split into sequence_len chunks)."""

    def tokenize(self, row):
        field = self.ds_cfg.get("field") or self.ds_cfg.get("text_column") or "text"
        ids = _tok(self.tok, row[field], add_bos=True, add_eos=True)
        out = []
        for i in range(0, len(ids), self.seq_len):
            chunk = ids[i:i + self.seq_len]
            out.append(_pack(chunk, chunk))
        return out


class PretrainStrategy(CompletionStrategy):
    pass


class InputOutputStrategy(Strategy):
    """``segments: [{text, label: bool}]`` -- template-free masking."""

    def tokenize(self, row):
        ids, labels = [], []
        segs = row["segments"]
        for i, seg in enumerate(segs):
            t = _tok(self.tok, seg["text"], add_bos=(i == 0), add_eos=False)
            ids += t
            labels += t if (seg.get("label") or self.train_on_inputs) else [IGNORE_INDEX] * len(t)
        ids, labels = ids[:self.seq_len], labels[:self.seq_len]
        return _pack(ids, labels)


class PretokenizedStrategy(Strategy):
    def tokenize(self, row):
        ids = list(row["input_ids"])[: self.seq_len]
        labels = list(row.get("labels", ids))[: self.seq_len]
        return _pack(ids, labels)


class StepwiseSupervisedStrategy(Strategy):
    """Process-reward data: prompt + completions[] + labels[]; the label of each step sits on the
    step separator token."""

    def tokenize(self, row):
        sep = self.ds_cfg.get("step_separator") or "\n"
        ids = _tok(self.tok, row["prompt"], add_bos=True)
        labels = [IGNORE_INDEX] * len(ids)
        for step, lab in zip(row["completions"], row["labels"]):
            t = _tok(self.tok, step + sep, add_bos=False)
            ids += t
            labels += [IGNORE_INDEX] * (len(t) - 1) + [int(bool(lab))]
        return _pack(ids[: self.seq_len], labels[: self.seq_len])


class BradleyTerryStrategy(Strategy):
    """Reward-model pairs: returns chosen/rejected token ids."""

    def tokenize(self, row):
        sys_ = row.get("system", "")
        prompt = (sys_ + "\n" if sys_ else "") + row.get("input", row.get("prompt", ""))
        c = _tok(self.tok, prompt + row["chosen"], add_eos=True, max_len=self.seq_len)
        r = _tok(self.tok, prompt + row["rejected"], add_eos=True, max_len=self.seq_len)
        return {"input_ids_chosen": c, "attention_mask_chosen": [1] * len(c),
                "input_ids_rejected": r, "attention_mask_rejected": [1] * len(r)}


def _late_registry():
    """Strategies that live in their own modules (they import this one)."""
    from .chat_template import ChatTemplateStrategy, MessagesStrategy
    from .strategies_extra import EXTRA

    out = {"chat_template": ChatTemplateStrategy, "messages": MessagesStrategy, "messages.chat": MessagesStrategy,
           "sharegpt": ChatTemplateStrategy}
    out.update(EXTRA)
    return out


_REGISTRY = {
    "alpaca": AlpacaStrategy, "alpaca:chat": AlpacaChatStrategy, "alpaca_chat": AlpacaChatStrategy,
    "alpaca:instruct": AlpacaStrategy, "gpteacher": GPTeacherStrategy, "oasst": OpenAssistantStrategy,
    "jeopardy": JeopardyStrategy, "summarizetldr": SummarizeTLDRStrategy, "completion": CompletionStrategy,
    "pretrain": PretrainStrategy, "input_output": InputOutputStrategy, "user_defined": UserDefinedStrategy,
    "stepwise_supervised": StepwiseSupervisedStrategy, "bradley_terry": BradleyTerryStrategy,
    "bradley_terry.chat_template": BradleyTerryStrategy, "pretokenized": PretokenizedStrategy,
}


def register_strategy(name, cls):
    _REGISTRY[name] = cls


def load_strategy(type_, tokenizer, cfg, ds_cfg=None):
    """``type`` may be a name, ``module.function`` of a user module, or a dict (user_defined)."""
    if isinstance(type_, dict):
        return UserDefinedStrategy(tokenizer, cfg, ds_cfg)
    if type_ is None:
        return PretokenizedStrategy(tokenizer, cfg, ds_cfg)
    if type_ not in _REGISTRY:
        for k, v in _late_registry().items():
            _REGISTRY.setdefault(k, v)
    if type_ in _REGISTRY:
        return _REGISTRY[type_](tokenizer, cfg, ds_cfg)
    if "." in type_:
        import importlib

        mod, _, fn = type_.rpartition(".")
        try:
            obj = getattr(importlib.import_module(mod), fn)
            return obj(tokenizer, cfg, ds_cfg)
        except (ImportError, AttributeError):
            pass
    raise ValueError(f"unknown dataset type '{type_}' (have: {sorted(_REGISTRY)})")


def is_pretokenized(columns) -> bool:
    return "input_ids" in columns and "labels" in columns or ("input_ids" in columns and "attention_mask" in columns)
