"""``type: chat_template``: conversations rendered with a Jinja chat template and masked turn by turn.

Semantics restated from the reference (src/axolotl/prompt_strategies/chat_template.py:278-1086,
src/axolotl/prompt_strategies/jinja_template_analyzer.py):

* A conversation is a list of messages; property mappings, role aliases, a row-level ``system`` field,
  ``drop_system_message`` and ``split_thinking`` (``<think>…</think>`` moved into the template's thinking
  key) are applied first. Extra message keys survive only if the template reads them (found by walking
  the template's syntax tree, see ``template_message_variables``).
* All labels start at -100. A turn is trained if its ``training`` field says so, else if it carries a
  ``training_detail``, else if ``train_on_inputs`` or its role is in ``roles_to_train``.
* The token span of a turn's CONTENT is located by rendering the conversation up to that turn twice — once
  with the content replaced by a dummy string — and taking the first and last differing token
  (``find_turn``); template headers and generation prompts therefore never receive labels.
* ``training_detail`` (character offsets with a train flag, or content given as a list of parts with
  ``train`` / ``weight``) selects tokens inside the span; a token that straddles a boundary is masked.
* The first EOT / EOS token within three tokens after the span follows ``train_on_eot`` /
  ``train_on_eos`` ∈ {``turn`` (with its turn), ``all``, ``last`` (only the final one), ``none``}.
"""
from __future__ import annotations

import json

from ..utils.logging import get_logger
from .strategies import IGNORE_INDEX, Strategy, _pack

LOG = get_logger(__name__)

DEFAULT_ROLES = {"human": "user", "user": "user", "assistant": "assistant", "gpt": "assistant", "system": "system",
                 "tool": "tool"}
THINKING_PAIRS = (("<think>", "</think>"), ("<reasoning>", "</reasoning>"), ("<|begin_of_thought|>", "<|end_of_thought|>"))
SOLUTION_PAIRS = (("<|begin_of_solution|>", "<|end_of_solution|>"),)


def template_message_variables(template: str, messages_name: str = "messages") -> set[str]:
    """Names of the per-message fields a chat template reads: every ``m.field`` / ``m['field']`` where ``m``
    is the loop variable of a ``for m in messages`` (or an alias assigned from it, or ``messages[i]``)."""
    try:
        import jinja2
        from jinja2 import nodes
    except ImportError:   # pragma: no cover
        return {"role", "content"}
    try:
        tree = jinja2.Environment(extensions=["jinja2.ext.loopcontrols"]).parse(template)
    except jinja2.TemplateSyntaxError:
        return {"role", "content"}
    msg_lists, msg_vars, found = {messages_name}, set(), set()

    def is_list(n):
        if isinstance(n, nodes.Name):
            return n.name in msg_lists
        if isinstance(n, nodes.Getitem) and isinstance(n.arg, nodes.Slice):
            return is_list(n.node)
        if isinstance(n, nodes.Filter):
            return n.node is not None and is_list(n.node)
        return False

    def is_msg(n):
        if isinstance(n, nodes.Name):
            return n.name in msg_vars
        if isinstance(n, nodes.Getitem) and not isinstance(n.arg, nodes.Slice):
            return is_list(n.node)
        return False

    for _ in range(3):   # aliases can be chained: a few passes reach the fixed point
        for n in tree.find_all((nodes.For, nodes.Assign)):
            if isinstance(n, nodes.For) and isinstance(n.target, nodes.Name) and is_list(n.iter):
                msg_vars.add(n.target.name)
            elif isinstance(n, nodes.Assign) and isinstance(n.target, nodes.Name):
                if is_msg(n.node):
                    msg_vars.add(n.target.name)
                elif is_list(n.node):
                    msg_lists.add(n.target.name)
    for n in tree.find_all((nodes.Getattr, nodes.Getitem)):
        if isinstance(n, nodes.Getattr) and is_msg(n.node):
            found.add(n.attr)
        elif isinstance(n, nodes.Getitem) and is_msg(n.node) and isinstance(n.arg, nodes.Const) and isinstance(n.arg.value, str):
            found.add(n.arg.value)
    # `'field' in message` tests
    for n in tree.find_all(nodes.Compare):
        for op in n.ops:
            if op.op in ("in", "notin") and is_msg(op.expr) and isinstance(n.expr, nodes.Const) and isinstance(n.expr.value, str):
                found.add(n.expr.value)
    return found or {"role", "content"}


def convert_content_parts(content):
    """Content given as a list of parts -> (text, training_detail or None). A part is ``{text|content|value,
    train?: bool, weight?: 0|1}``; offsets are character positions in the concatenated text."""
    if not isinstance(content, list):
        return None
    texts, details, explicit, off = [], [], False, 0
    for part in content:
        if not isinstance(part, dict):
            continue
        text = part.get("text") or part.get("content") or part.get("value") or ""
        texts.append(text)
        tr, wt = part.get("train"), part.get("weight")
        if tr is not None or wt is not None:
            explicit = True
            train = tr if tr is not None else (wt not in (0, 0.0))
        else:
            train = True
        if text:
            details.append({"begin_offset": off, "end_offset": off + len(text) - 1, "train": bool(train)})
            off += len(text)
    if explicit:
        for i in range(len(details) - 1):
            if details[i]["train"] != details[i + 1]["train"] and texts[i] and texts[i][-1] in (" ", "\t"):
                LOG.warning("content part %d ends with whitespace at a train/mask boundary; the space merges with the "
                            "next part's first token, which is then masked. Move it to the start of the next part.", i)
    return "".join(texts), (details if explicit else None)


class ChatTemplateStrategy(Strategy):
    def __init__(self, tokenizer, cfg, ds_cfg=None):
        super().__init__(tokenizer, cfg, ds_cfg)
        d = self.ds_cfg
        self.field_messages = d.get("field_messages") or "messages"
        self.field_system = d.get("field_system") or "system"
        self.field_tools = d.get("field_tools") or "tools"
        self.thinking_key = d.get("template_thinking_key") or "reasoning_content"
        mp = dict(d.get("message_property_mappings") or {})
        if not mp:
            mp = {"role": d.get("message_field_role") or "role", "content": d.get("message_field_content") or "content"}
            mp[self.thinking_key] = d.get("field_thinking") or "reasoning_content"
        self.mappings = mp
        self.f_training = d.get("message_field_training") or "training"
        self.f_training_detail = d.get("message_field_training_detail") or "training_detail"
        self.roles_to_train = d.get("roles_to_train") if d.get("roles_to_train") is not None else ["assistant"]
        self.train_on_eos = d.get("train_on_eos") or "turn"
        self.split_thinking = bool(d.get("split_thinking"))
        self.drop_system = bool(d.get("drop_system_message"))
        self.role_map = dict(DEFAULT_ROLES)
        if d.get("roles"):
            self.role_map = {src: canon for canon, names in d["roles"].items() for src in names}
        self.kwargs = dict(cfg.get("chat_template_kwargs") or d.get("chat_template_kwargs") or {})
        self.template = self._resolve_template(d)
        self.msg_vars = template_message_variables(self.template or "", "messages")
        # ---- end-of-turn tokens
        eot = d.get("eot_tokens") or cfg.get("eot_tokens")
        self.eot_tokens = list(eot) if eot else ([tokenizer.eos_token] if tokenizer.eos_token else [])
        self.train_on_eot = d.get("train_on_eot") or self.train_on_eos
        self.eot_ids = set()
        for t in self.eot_tokens:
            ids = tokenizer.encode(t, add_special_tokens=False)
            if len(ids) == 1:
                self.eot_ids.add(ids[0])
            elif eot and self.template and t in self.template:
                raise ValueError(f"EOT token '{t}' is encoded as multiple tokens: {ids}. Please add it under `tokens: ` in "
                                 "the config or (recommended) override unused added_tokens via `added_tokens_overrides: `.")
        if eot and tokenizer.eos_token in self.eot_tokens and self.train_on_eos != self.train_on_eot:
            raise ValueError("Conflict between train_on_eos and train_on_eot. eos_token is in eot_tokens and "
                             f"train_on_eos != train_on_eot (train_on_eos: {self.train_on_eos}, train_on_eot: {self.train_on_eot})")
        if self.template and tokenizer.eos_token and not eot and tokenizer.eos_token not in self.template \
                and "eos_token" not in self.template:
            LOG.warning("EOS token %r not found in chat_template; the turn terminator won't be trained. Set `eot_tokens` "
                        "to your template's turn-ending token.", tokenizer.eos_token)

    def _resolve_template(self, d):
        from .tokenizer import get_chat_template

        name = d.get("chat_template") or self.cfg.get("chat_template")
        jinja = d.get("chat_template_jinja") or self.cfg.get("chat_template_jinja")
        if name or jinja:
            return get_chat_template(name or "jinja", self.tok, jinja)
        return getattr(self.tok, "chat_template", None)

    # ------------------------------------------------------------------ rendering
    def render(self, turns, add_generation_prompt=False, tools=None, real_last_index=None):
        kw = dict(self.kwargs)
        if self.template:
            kw["chat_template"] = self.template
        if tools:
            kw["tools"] = tools
        if real_last_index:
            kw["real_last_index"] = real_last_index
        clean = [{k: v for k, v in t.items() if k not in ("training", "training_detail", "reasoning_training_detail")}
                 for t in turns]
        out = self.tok.apply_chat_template(clean, tokenize=True, add_generation_prompt=add_generation_prompt, **kw)
        if isinstance(out, dict) or hasattr(out, "keys"):
            out = out["input_ids"]
        return list(out)

    # ------------------------------------------------------------------ conversation
    def transform_message(self, m):
        out = {}
        for key, src in self.mappings.items():
            if m.get(src) is not None:
                out[key] = m[src]
        if "role" not in out and m.get("from") is not None:      # sharegpt spelling
            out["role"] = m["from"]
        if "content" not in out and m.get("value") is not None:
            out["content"] = m["value"]
        if "role" in out:
            out["role"] = self.role_map.get(out["role"], out["role"])
        if self.split_thinking and out.get("role") == "assistant" and isinstance(out.get("content"), str):
            content = out["content"]
            for a, b in THINKING_PAIRS:
                if a in content and b in content:
                    i, j = content.find(a), content.find(b)
                    out[self.thinking_key] = content[i + len(a):j].strip()
                    rest = content[j + len(b):].lstrip()
                    for ca, cb in SOLUTION_PAIRS:
                        if ca in rest and cb in rest:
                            rest = rest[rest.find(ca) + len(ca):rest.find(cb)].strip()
                            break
                    out["content"] = rest
                    break
        mapped = set(self.mappings.values()) | {"from", "value"}
        for key in self.msg_vars:
            if key in m and key not in mapped and key not in out and m[key] is not None:
                out[key] = m[key]
        for call in out.get("tool_calls") or []:
            fn = call.get("function") if isinstance(call, dict) else None
            if fn and isinstance(fn.get("arguments"), str):
                try:
                    fn["arguments"] = json.loads(fn["arguments"])
                except json.JSONDecodeError as exc:
                    raise ValueError(f"tool_calls arguments of function {fn.get('name', 'unknown')!r} are not valid JSON: "
                                     f"{fn['arguments']!r}") from exc
        return out

    def conversation(self, row):
        msgs = row.get(self.field_messages) or row.get("conversations") or []
        if not msgs:
            return []
        turns = []
        first = self.transform_message(msgs[0])
        if first.get("role") != "system" and row.get(self.field_system):
            turns.append({"role": "system", "content": row[self.field_system]})
        for m in msgs:
            t = self.transform_message(m)
            if m.get(self.f_training) is not None:
                t["training"] = m[self.f_training]
            if m.get(self.f_training_detail) is not None:
                t["training_detail"] = m[self.f_training_detail]
            conv = convert_content_parts(t.get("content"))
            if conv is not None:
                t["content"] = conv[0]
                if conv[1] is not None:
                    t["training_detail"] = conv[1]
            if self.thinking_key in t:
                conv = convert_content_parts(t[self.thinking_key])
                if conv is not None:
                    t[self.thinking_key] = conv[0]
                    if conv[1] is not None:
                        t["reasoning_training_detail"] = conv[1]
            turns.append(t)
        if self.drop_system and turns and turns[0].get("role") == "system":
            turns = turns[1:]
        return turns

    # ------------------------------------------------------------------ span location
    def find_turn(self, turns, idx, tools=None, content_only=False, reasoning_only=False):
        """(start, end) token positions of turn ``idx``'s content inside the rendering of ``turns[:idx + 1]``,
        or (-1, -1) when the template does not emit it."""
        turn = turns[idx]
        name = str(getattr(self.tok, "name_or_path", "")).lower()
        if idx == 0 and turn.get("role") == "system" and "mistral" in name:
            return -1, -1     # Mistral templates fold a lone system message into the next user turn
        if reasoning_only:
            dummy = {"role": turn.get("role"), "content": turn.get("content", "")}
            if self.thinking_key in turn:
                dummy[self.thinking_key] = "[[dummy_reasoning]]"
        else:
            dummy = {"role": turn.get("role"), "content": "[[dummy_message]]"}
            if content_only and self.thinking_key in turn:
                dummy[self.thinking_key] = turn[self.thinking_key]
        last = len(turns) - 1
        a = self.render(turns[:idx] + [dummy], tools=tools, real_last_index=last)
        b = self.render(turns[:idx + 1], tools=tools, real_last_index=last)
        if not a or not b:
            return -1, -1
        n = min(len(a), len(b))
        start = next((i for i in range(n) if a[i] != b[i]), None)
        if start is None:
            return -1, -1
        end = next((len(b) - i for i in range(n) if a[len(a) - 1 - i] != b[len(b) - 1 - i]), None)
        if end is None or end <= start:
            return -1, -1
        return start, end

    def detail_token_mask(self, text, details):
        """One flag per token of ``text``: True where the token lies completely inside a ``train: true`` range
        (after snapping the ranges outwards to token boundaries); straddling tokens stay masked."""
        enc = self.tok(text, return_offsets_mapping=True, add_special_tokens=False)
        offs = [list(o) for o in enc["offset_mapping"]]
        if not offs:
            return []
        for i in range(len(offs) - 1):
            offs[i][1] = offs[i + 1][0] - 1
        offs[-1][1] = len(text) - 1
        adjusted = []
        for dtl in details:
            b0, e0 = dtl["begin_offset"], dtl["end_offset"]
            bt = next((i for i, (s, e) in enumerate(offs) if s >= b0), len(offs))
            if bt > 0 and offs[bt - 1][1] > b0:
                bt -= 1
            et = next((i for i in range(len(offs) - 1, -1, -1) if offs[i][1] <= e0), -1)
            if et < len(offs) - 1 and offs[et + 1][0] < e0:
                et += 1
            if bt <= et and bt < len(offs):
                adjusted.append((offs[bt][0], offs[et][1], bool(dtl.get("train", True))))
        mask = [False] * len(offs)
        for i, (s, e) in enumerate(offs):
            for (b0, e0, tr) in adjusted:
                if s >= b0 and e <= e0 and tr:
                    mask[i] = True
        return mask

    # ------------------------------------------------------------------ tokenisation
    def tokenize(self, row):
        turns = self.conversation(row)
        if not turns:
            return None
        tools = row.get(self.field_tools)
        if isinstance(tools, str):
            tools = json.loads(tools)
        ids = self.render(turns, tools=tools)
        labels = [IGNORE_INDEX] * len(ids)
        last_eot = last_eos = -1
        eos_id = self.tok.eos_token_id
        for i, turn in enumerate(turns):
            detail, rdetail = turn.get("training_detail"), turn.get("reasoning_training_detail")
            if turn.get("training") is not None:
                train = bool(turn["training"])
            elif detail is not None or rdetail is not None:
                train = bool(detail) or bool(rdetail)
            else:
                train = self.train_on_inputs or turn.get("role") in self.roles_to_train
            if not train and self.train_on_eos != "all" and self.train_on_eot != "all":
                if i == len(turns) - 1:
                    LOG.debug("last turn is not trainable: its EOS / EOT token stays masked")
                continue
            has_reasoning = turn.get(self.thinking_key) is not None
            start, end = self.find_turn(turns, i, tools, content_only=bool((detail or rdetail) and has_reasoning))
            if train and start != -1:
                if detail:
                    if not isinstance(turn.get("content"), str):
                        raise ValueError("`train_detail` is not supported when `content` is not a string.")
                    for k, on in enumerate(self.detail_token_mask(turn["content"], detail)):
                        if on and start + k < len(ids):
                            labels[start + k] = ids[start + k]
                elif not rdetail:
                    labels[start:end] = ids[start:end]
            if train and rdetail and has_reasoning:
                rs, re_ = self.find_turn(turns, i, tools, reasoning_only=True)
                if rs != -1:
                    for k, on in enumerate(self.detail_token_mask(turn[self.thinking_key], rdetail)):
                        if on and rs + k < len(ids):
                            labels[rs + k] = ids[rs + k]
            if end == -1:
                continue
            for kind, wanted, option in (("eot", self.eot_ids, self.train_on_eot), ("eos", {eos_id}, self.train_on_eos)):
                pos = next((j for j in range(end, len(ids)) if ids[j] in wanted), -1)
                if pos != -1 and abs(pos - end) <= 3:      # template padding between content and terminator
                    if kind == "eot":
                        last_eot = pos
                    else:
                        last_eos = pos
                    if option == "all" or (option == "turn" and train):
                        labels[pos] = ids[pos]
        for pos, option in ((last_eot, self.train_on_eot), (last_eos, self.train_on_eos)):
            if option == "last" and pos != -1:
                labels[pos] = ids[pos]
        return _pack(ids[: self.seq_len], labels[: self.seq_len])


class MessagesStrategy(ChatTemplateStrategy):
    """``type: messages`` — OpenAI-style rows; the same masking with the tokenizer's own template."""
