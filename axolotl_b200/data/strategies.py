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


class ChatTemplateStrategy(Strategy):
    def __init__(self, tokenizer, cfg, ds_cfg=None):
        super().__init__(tokenizer, cfg, ds_cfg)
        d = self.ds_cfg
        self.field_messages = d.get("field_messages") or "messages"
        mp = d.get("message_property_mappings") or {}
        self.f_role = mp.get("role") or d.get("message_field_role") or "role"
        self.f_content = mp.get("content") or d.get("message_field_content") or "content"
        self.f_training = d.get("message_field_training") or "training"
        self.roles_to_train = d.get("roles_to_train") if d.get("roles_to_train") is not None else ["assistant"]
        self.train_on_eos = d.get("train_on_eos") or "turn"
        self.train_on_eot = d.get("train_on_eot") or self.train_on_eos
        self.role_map = {"human": "user", "gpt": "assistant", "system": "system", "user": "user",
                         "assistant": "assistant", "tool": "tool", "ipython": "ipython"}
        for canon, names in (d.get("roles") or {}).items():
            for n in names:
                self.role_map[n] = canon
        eot = cfg.get("eot_tokens") or []
        self.eot_ids = {tokenizer.convert_tokens_to_ids(t) for t in eot}
        if tokenizer.eos_token_id is not None:
            self.eot_ids.add(tokenizer.eos_token_id)
        self.drop_system = bool(d.get("drop_system_message"))

    def _messages(self, row):
        msgs = row.get(self.field_messages) or row.get("conversations") or []
        out = []
        for m in msgs:
            role = m.get(self.f_role, m.get("from"))
            content = m.get(self.f_content, m.get("value", ""))
            role = self.role_map.get(role, role)
            if role == "system" and self.drop_system:
                continue
            o = {"role": role, "content": content}
            if self.f_training in m:
                o["training"] = m[self.f_training]
            out.append(o)
        return out

    def _render(self, msgs, add_generation_prompt=False, tools=None):
        clean = [{"role": m["role"], "content": m["content"]} for m in msgs]
        kw = dict(self.cfg.get("chat_template_kwargs") or {})
        out = self.tok.apply_chat_template(clean, tokenize=True, add_generation_prompt=add_generation_prompt,
                                           tools=tools, **kw)
        if isinstance(out, dict):
            out = out["input_ids"]
        return list(out)

    def tokenize(self, row):
        msgs = self._messages(row)
        if not msgs:
            return None
        tools = row.get(self.ds_cfg.get("field_tools") or "tools")
        full = self._render(msgs, tools=tools)
        labels = [IGNORE_INDEX] * len(full)
        last_trainable = None
        prev_len = 0
        for i, m in enumerate(msgs):
            upto = self._render(msgs[: i + 1], tools=tools)
            # the rendered prefix must be a prefix of the full rendering; otherwise fall back to lengths
            end = min(len(upto), len(full))
            start = prev_len
            if m["role"] == "assistant" and i > 0:
                # skip the generation prompt (header tokens of the assistant turn)
                gen = self._render(msgs[:i], add_generation_prompt=True, tools=tools)
                if len(gen) <= end and gen == full[: len(gen)]:
                    start = len(gen)
            trainable = m.get("training")
            if trainable is None:
                trainable = self.train_on_inputs or (m["role"] in self.roles_to_train)
            if trainable:
                for j in range(start, end):
                    labels[j] = full[j]
                last_trainable = (start, end)
                if self.train_on_eos == "none" or self.train_on_eot == "none":
                    for j in range(start, end):
                        if full[j] in self.eot_ids:
                            labels[j] = IGNORE_INDEX
            elif self.train_on_eos == "all" or self.train_on_eot == "all":
                for j in range(start, end):
                    if full[j] in self.eot_ids:
                        labels[j] = full[j]
            prev_len = end
        if self.train_on_eos == "last" and last_trainable is not None:
            s, e = last_trainable
            for j in range(len(full)):
                if full[j] in self.eot_ids and not (s <= j < e):
                    labels[j] = IGNORE_INDEX if labels[j] != IGNORE_INDEX and j < s else labels[j]
        full, labels = full[: self.seq_len], labels[: self.seq_len]
        return _pack(full, labels)


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


_REGISTRY = {
    "alpaca": AlpacaStrategy, "alpaca:chat": AlpacaChatStrategy, "alpaca_chat": AlpacaChatStrategy,
    "alpaca:instruct": AlpacaStrategy, "gpteacher": GPTeacherStrategy, "oasst": OpenAssistantStrategy,
    "jeopardy": JeopardyStrategy, "summarizetldr": SummarizeTLDRStrategy, "completion": CompletionStrategy,
    "pretrain": PretrainStrategy, "input_output": InputOutputStrategy, "chat_template": ChatTemplateStrategy,
    "messages": ChatTemplateStrategy, "sharegpt": ChatTemplateStrategy, "user_defined": UserDefinedStrategy,
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
