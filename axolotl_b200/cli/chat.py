"""Multi-turn chat REPL on a model + adapter described by a training config.

Slash commands: ``/system <text>`` sets the system prompt, ``/reset`` clears the history,
``/temp <t>``, ``/max <n>`` change sampling, ``/undo`` drops the last exchange, ``/save <file>``
writes the conversation as JSON, ``/exit`` leaves. The conversation is rendered with the
tokenizer's (or the configured) chat template at every turn.
Reference: src/axolotl/cli/chat.py (REPL) and cli/inference.py.
"""
from __future__ import annotations

import json

import torch


class ChatSession:
    def __init__(self, model, tokenizer, system=None, max_new_tokens=256, temperature=0.7, top_p=0.95):
        self.model, self.tok = model, tokenizer
        self.system, self.history = system, []
        self.max_new_tokens, self.temperature, self.top_p = max_new_tokens, temperature, top_p

    def messages(self):
        msgs = [{"role": "system", "content": self.system}] if self.system else []
        return msgs + self.history

    def _prompt_ids(self):
        if getattr(self.tok, "chat_template", None):
            ids = self.tok.apply_chat_template(self.messages(), tokenize=True, add_generation_prompt=True)
            return list(ids["input_ids"] if isinstance(ids, dict) else ids)
        text = "".join(f"{m['role']}: {m['content']}\n" for m in self.messages()) + "assistant: "
        return list(self.tok(text)["input_ids"])

    def command(self, line):
        """Handles a slash command; returns a status string, or None if ``line`` is not one."""
        if not line.startswith("/"):
            return None
        cmd, _, arg = line[1:].partition(" ")
        if cmd == "system":
            self.system = arg.strip() or None
            return "system prompt set" if self.system else "system prompt cleared"
        if cmd == "reset":
            self.history = []
            return "history cleared"
        if cmd == "undo":
            while self.history and self.history[-1]["role"] != "user":
                self.history.pop()
            if self.history:
                self.history.pop()
            return "last exchange removed"
        if cmd == "temp":
            self.temperature = float(arg)
            return f"temperature = {self.temperature}"
        if cmd == "max":
            self.max_new_tokens = int(arg)
            return f"max_new_tokens = {self.max_new_tokens}"
        if cmd == "save":
            with open(arg.strip(), "w") as fh:
                json.dump(self.messages(), fh, indent=2)
            return f"saved to {arg.strip()}"
        if cmd in ("exit", "quit"):
            raise EOFError
        return f"unknown command /{cmd}"

    def say(self, text):
        self.history.append({"role": "user", "content": text})
        ids = self._prompt_ids()
        dev = self.model.embed_tokens.device
        out = self.model.generate(torch.tensor([ids], device=dev), max_new_tokens=self.max_new_tokens,
                                  temperature=self.temperature, top_p=self.top_p,
                                  eos_token_id=getattr(self.tok, "eos_token_id", None))
        new = out[0].tolist()[len(ids):]
        reply = self.tok.decode(new, skip_special_tokens=True)
        self.history.append({"role": "assistant", "content": reply})
        return reply


def run_repl(cfg, system=None, max_new_tokens=256, temperature=0.7, input_fn=input, echo=print):
    from ..data.tokenizer import load_tokenizer
    from ..train.evaluate import _device
    from ..train.run import build_model, setup_adapter

    tok = load_tokenizer(cfg)
    model = build_model(cfg, _device(cfg))
    setup_adapter(cfg, model)
    model.eval()
    sess = ChatSession(model, tok, system, max_new_tokens, temperature)
    echo("chat ready: /system /reset /undo /temp /max /save /exit")
    while True:
        try:
            line = input_fn("> ").strip()
            if not line:
                continue
            status = sess.command(line)
            echo(status if status is not None else sess.say(line))
        except (EOFError, KeyboardInterrupt):
            break
    return sess
