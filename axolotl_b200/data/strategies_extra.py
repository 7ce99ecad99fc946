"""Instruction / role-play formats with fixed prompt layouts (what the reference ships as
src/axolotl/prompt_strategies/{llama2_chat,metharme,orcamini,pygmalion,context_qa,creative_acr}.py)."""
from __future__ import annotations

from .strategies import IGNORE_INDEX, AlpacaStrategy, Strategy, _pack, _tok

LLAMA2_SYSTEM = ("You are a helpful, respectful and honest assistant. Always answer as helpfully as possible, while "
                 "being safe. Your answers should not include any harmful, unethical, racist, sexist, toxic, dangerous, or "
                 "illegal content. Please ensure that your responses are socially unbiased and positive in nature.\n\n"
                 "If a question does not make any sense, or is not factually coherent, explain why instead of answering "
                 "something not correct. If you don't know the answer to a question, please don't share false information.")


class Llama2ChatStrategy(Strategy):
    """``<s>[INST] <<SYS>>\\n{system}\\n<</SYS>>\\n\\n{user} [/INST] {assistant} </s><s>[INST] …``; only the
    assistant replies (and their closing ``</s>``) are trained. Rows are ShareGPT-style ``conversations``."""

    def tokenize(self, row):
        conv = row.get("conversations") or row.get("messages") or []
        system = row.get("system") or LLAMA2_SYSTEM
        turns = []
        for m in conv:
            role = m.get("from", m.get("role"))
            text = m.get("value", m.get("content", ""))
            if role == "system":
                system = text
            else:
                turns.append(("user" if role in ("human", "user") else "assistant", text))
        if turns and turns[0][0] == "assistant":
            turns = turns[1:]
        ids, labels = [], []
        first = True
        for k in range(0, len(turns) - 1, 2):
            (ru, user), (ra, reply) = turns[k], turns[k + 1]
            if ru != "user" or ra != "assistant":
                break
            head = f"[INST] <<SYS>>\n{system}\n<</SYS>>\n\n{user.strip()} [/INST]" if first else f"[INST] {user.strip()} [/INST]"
            first = False
            p = _tok(self.tok, head, add_bos=True)
            r = _tok(self.tok, " " + reply.strip() + " ", add_bos=False, add_eos=True)
            ids += p + r
            labels += (p if self.train_on_inputs else [IGNORE_INDEX] * len(p)) + r
        if not ids:
            return None
        return _pack(ids[: self.seq_len], labels[: self.seq_len])


class MetharmeStrategy(Strategy):
    """``prompt`` (already carrying ``<|system|>…<|user|>…<|model|>``) + ``generation``; the generation is
    trained and closed with up to three EOS tokens, as the Metharme recipe does."""

    def tokenize(self, row):
        p = _tok(self.tok, row["prompt"], add_bos=True, max_len=self.seq_len)
        r = _tok(self.tok, row["generation"], add_bos=False, add_eos=False)
        eos = self.tok.eos_token_id
        if eos is not None:
            r = r + [eos] * (3 - (1 if r and r[-1] == eos else 0))
        r = r[: max(self.seq_len - len(p), 0)]
        return _pack(p + r, (p if self.train_on_inputs else [IGNORE_INDEX] * len(p)) + r)


class OrcaMiniStrategy(AlpacaStrategy):
    def prompt_response(self, row):
        system, q = row.get("system_prompt", row.get("system", "")), row.get("question", row.get("instruction", ""))
        return f"### System:\n{system}\n\n### User:\n{q}\n\n### Response:\n", row.get("response", row.get("output", ""))


class PygmalionStrategy(Strategy):
    """``conversations`` of (system | human | bot): ``<|system|>Persona: …``, ``<|user|> …``, ``<|model|> …``;
    bot turns are trained except for their ``<|model|>`` prefix and end with EOS."""

    def tokenize(self, row):
        prefix = _tok(self.tok, "<|model|>", add_bos=False)
        ids, labels = [], []
        for m in row["conversations"]:
            role, text = m.get("role", m.get("from")), m.get("value", m.get("content", ""))
            if role == "system":
                if text.endswith("\n<START>"):
                    text = text[:-8]
                t = _tok(self.tok, "<|system|>Persona: " + text.strip(), add_bos=True)
                lab = [IGNORE_INDEX] * len(t)
            elif role in ("human", "user"):
                t = _tok(self.tok, "<|user|> " + text.strip(), add_bos=False)
                lab = [IGNORE_INDEX] * len(t)
            elif role in ("bot", "gpt", "assistant"):
                t = _tok(self.tok, "<|model|> " + text.strip(), add_bos=False, add_eos=True)
                lab = [IGNORE_INDEX] * len(prefix) + t[len(prefix):]
            else:
                continue
            ids += t
            labels += lab
        if not ids:
            return None
        return _pack(ids[: self.seq_len], labels[: self.seq_len])


class ContextQAStrategy(AlpacaStrategy):
    """``context`` + ``question`` -> ``answer`` (``context_qa.load_v2`` layout)."""

    def prompt_response(self, row):
        return ("Context: " + row.get("context", "") + "\nQuestion: " + row.get("question", "") + "\n",
                "Answer: " + row.get("answer", ""))


class ArticleQAStrategy(AlpacaStrategy):
    """``article`` + ``question`` -> ``answer`` in the Alpaca instruction layout (``context_qa.load``)."""

    def fields(self, row):
        return row.get("article", "") + "\n===\n" + row.get("question", ""), "", row.get("answer", "")


class UnanswerableQAStrategy(AlpacaStrategy):
    def fields(self, row):
        return (row.get("article", "") + "\n===\n" + row.get("unanswerable_question", ""), "",
                "The given information does not answer the question.")


class CreativeAnswerStrategy(AlpacaStrategy):
    """Creative-writing rows (``creative_acr.load_answer``): instruction -> answer."""

    def fields(self, row):
        return row.get("instruction", ""), "", row.get("answer", "")


class CreativeCritiqueStrategy(AlpacaStrategy):
    def fields(self, row):
        scores = "\n".join(f"{k}: {v}" for k, v in (row.get("scores") or {}).items())
        q = ("Critique the following answer to the instruction; score it on the listed criteria and explain.\n\n"
             f"Instruction:\n{row.get('instruction', '')}\n\nAnswer:\n{row.get('answer', '')}")
        return q, "", (scores + "\n\n" if scores else "") + row.get("critiques", row.get("critique", ""))


class CreativeReviseStrategy(AlpacaStrategy):
    def fields(self, row):
        q = ("Revise the answer to the instruction using the critique.\n\n"
             f"Instruction:\n{row.get('instruction', '')}\n\nAnswer:\n{row.get('answer', '')}\n\n"
             f"Critique:\n{row.get('critiques', row.get('critique', ''))}")
        return q, "", row.get("revision", "")


EXTRA = {
    "llama2_chat": Llama2ChatStrategy, "metharme": MetharmeStrategy, "orcamini": OrcaMiniStrategy,
    "pygmalion": PygmalionStrategy, "context_qa": ArticleQAStrategy, "context_qa.load_v2": ContextQAStrategy,
    "context_qa.load_404": UnanswerableQAStrategy, "creative_acr": CreativeAnswerStrategy,
    "creative_acr.load_answer": CreativeAnswerStrategy, "creative_acr.load_critique": CreativeCritiqueStrategy,
    "creative_acr.load_revise": CreativeReviseStrategy,
}
