"""Prompt strategies for preference data: raw row -> {prompt, chosen, rejected} (pairwise) or
{prompt, completion, label} (KTO) strings.

Names and field conventions mirror the reference's strategy modules so that dataset ``type:``
values carry over (src/axolotl/prompt_strategies/dpo/{chatml,llama3,zephyr,passthrough,
user_defined,chat_template}.py, .../kto/{chatml,llama3,user_defined}.py,
.../orpo/chat_template.py). The two chat dialects differ only in their turn delimiters, so one
table-driven builder covers both.
"""
from __future__ import annotations

_DIALECTS = {
    "chatml": dict(system="<|im_start|>system\n{}<|im_end|>\n", user="<|im_start|>user\n{}<|im_end|>\n",
                   gen="<|im_start|>assistant\n", end="<|im_end|>"),
    "llama3": dict(system="<|start_header_id|>system<|end_header_id|>\n\n{}<|eot_id|>",
                   user="<|start_header_id|>user<|end_header_id|>\n\n{}<|eot_id|>",
                   gen="<|start_header_id|>assistant<|end_header_id|>\n\n", end="<|eot_id|>"),
}


def _first(sample, keys):
    for k in keys:
        if k in sample:
            return sample[k]
    raise KeyError(f"none of {keys} in sample (has {list(sample)})")


def _content(v, idx):
    """A field that is either a string or a list of chat messages (take message ``idx``)."""
    return v[idx]["content"] if isinstance(v, (list, tuple)) else v


def _prompt(d, system, user):
    return (d["system"].format(system) if system else "") + d["user"].format(user) + d["gen"]


# variant -> (prompt keys, how to read the prompt, chosen keys, rejected keys, message index or None, use system)
_PAIR_VARIANTS = {
    "default": (("prompt", "input", "question", "instruction"), ("chosen", "chosen_response"),
                ("rejected", "rejected_response"), None, True),
    "icr": (("input",), ("chosen",), ("rejected",), None, True),
    "intel": (("question",), ("chosen",), ("rejected",), None, True),
    "prompt_pairs": (("prompt",), ("chosen",), ("rejected",), None, True),
    "ultra": (("prompt",), ("chosen",), ("rejected",), 1, True),
    "argilla_chat": (None, ("chosen",), ("rejected",), 1, False),
}

_KTO_VARIANTS = {
    "argilla": (("instruction",), None, True),
    "intel": (("question",), None, True),
    "prompt_pairs": (("prompt",), None, True),
    "ultra": (("prompt",), None, True),
    "argilla_chat": (None, 1, False),
}


def _pair_transform(dialect, variant):
    d = _DIALECTS[dialect]
    pkeys, ckeys, rkeys, midx, use_sys = _PAIR_VARIANTS[variant]

    def fn(sample):
        chosen, rejected = _first(sample, ckeys), _first(sample, rkeys)
        user = _content(chosen, 0) if pkeys is None else _first(sample, pkeys)
        system = sample.get("system") if use_sys else None
        return {"prompt": _prompt(d, system, user),
                "chosen": _content(chosen, midx if midx is not None else 0) + d["end"],
                "rejected": _content(rejected, midx if midx is not None else 0) + d["end"]}

    return fn


def _kto_transform(dialect, variant):
    d = _DIALECTS[dialect]
    pkeys, midx, use_sys = _KTO_VARIANTS[variant]

    def fn(sample):
        comp = sample["completion"]
        user = _content(comp, 0) if pkeys is None else _first(sample, pkeys)
        system = sample.get("system") if use_sys else None
        return {"prompt": _prompt(d, system, user), "completion": _content(comp, midx or 0) + d["end"],
                "label": bool(sample.get("label", True))}

    return fn


def _zephyr_nectar(sample):
    answers = sorted(sample["answers"], key=lambda a: a["rank"])
    return {"prompt": f"<|system|>\n</s>\n<|user|>\n{sample['prompt']}</s>\n<|assistant|>\n",
            "chosen": answers[-1]["answer"], "rejected": answers[-2]["answer"]}


def _user_defined(ds_type: dict, kto=False):
    f_prompt = ds_type.get("field_prompt", "prompt")
    f_system = ds_type.get("field_system", "system")
    p_fmt = ds_type.get("prompt_format") or "{prompt}"

    def prompt_of(sample):
        if "{system}" in p_fmt:
            return p_fmt.format(system=sample.get(f_system) or "", prompt=sample[f_prompt])
        return p_fmt.format(prompt=sample[f_prompt])

    if kto:
        f_comp, f_label = ds_type.get("field_completion", "completion"), ds_type.get("field_label", "label")
        c_fmt = ds_type.get("completion_format") or "{completion}"
        return lambda s: {"prompt": prompt_of(s), "completion": c_fmt.format(completion=s[f_comp]),
                          "label": bool(s[f_label])}
    f_c, f_r = ds_type.get("field_chosen", "chosen"), ds_type.get("field_rejected", "rejected")
    c_fmt = ds_type.get("chosen_format") or "{chosen}"
    r_fmt = ds_type.get("rejected_format") or "{rejected}"
    return lambda s: {"prompt": prompt_of(s), "chosen": c_fmt.format(chosen=s[f_c]),
                      "rejected": r_fmt.format(rejected=s[f_r])}


def _chat_template_pair(tokenizer, ds_cfg):
    """Messages + chosen/rejected answers rendered through the tokenizer's chat template
    (reference: prompt_strategies/dpo/chat_template.py, orpo/chat_template.py)."""
    f_msgs = ds_cfg.get("field_messages") or "messages"
    f_c, f_r = ds_cfg.get("field_chosen") or "chosen", ds_cfg.get("field_rejected") or "rejected"
    mp = ds_cfg.get("message_property_mappings") or {}
    k_role, k_content = mp.get("role", "role"), mp.get("content", "content")
    roles = {"human": "user", "gpt": "assistant"}
    for canon, names in (ds_cfg.get("roles") or {}).items():
        for n in names:
            roles[n] = canon

    def norm(m):
        return {"role": roles.get(m[k_role], m[k_role]), "content": m[k_content]}

    def answer(v):
        if isinstance(v, (list, tuple)):     # full conversation: the answer is its last message
            return norm(v[-1])["content"]
        if isinstance(v, dict):
            return v[k_content]
        return v

    def fn(sample):
        if f_msgs in sample:
            msgs = [norm(m) for m in sample[f_msgs]]
        elif isinstance(sample.get(f_c), (list, tuple)):
            msgs = [norm(m) for m in sample[f_c][:-1]]
        else:
            msgs = ([{"role": "system", "content": sample["system"]}] if sample.get("system") else []) + \
                [{"role": "user", "content": _first(sample, ("prompt", "question", "instruction", "input"))}]
        prompt = tokenizer.apply_chat_template(msgs, tokenize=False, add_generation_prompt=True)
        out = {}
        for name, key in (("chosen", f_c), ("rejected", f_r)):
            full = tokenizer.apply_chat_template(msgs + [{"role": "assistant", "content": answer(sample[key])}],
                                                 tokenize=False)
            out[name] = full[len(prompt):] if full.startswith(prompt) else answer(sample[key])
        out["prompt"] = prompt
        return out

    return fn


def load_preference_transform(ds_type, rl: str, tokenizer=None, ds_cfg=None):
    """``ds_type``: 'chatml.intel', 'llama3.ultra', 'zephyr.nectar', 'chat_template.default',
    'passthrough', a user-defined dict, or None (rows already hold the canonical fields)."""
    kto = rl == "kto"
    if ds_type is None or ds_type in ("passthrough", "passthrough.default"):
        return lambda s: s
    if isinstance(ds_type, dict):
        return _user_defined(ds_type, kto)
    base, _, variant = ds_type.partition(".")
    variant = variant or "default"
    if base in ("chat_template",):
        if tokenizer is None:
            raise ValueError("chat_template preference strategies need a tokenizer with a chat template")
        return _chat_template_pair(tokenizer, ds_cfg or {})
    if base == "zephyr" and variant == "nectar":
        return _zephyr_nectar
    if base == "user_defined":
        return _user_defined(ds_cfg.get("type") if isinstance((ds_cfg or {}).get("type"), dict) else {}, kto)
    if base in _DIALECTS:
        table = _KTO_VARIANTS if kto else _PAIR_VARIANTS
        if variant not in table:
            raise ValueError(f"unknown {rl} strategy '{ds_type}' (variants: {sorted(table)})")
        return (_kto_transform if kto else _pair_transform)(base, variant)
    raise ValueError(f"unknown preference dataset type '{ds_type}'")
