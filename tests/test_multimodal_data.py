"""Multimodal data path: role masking over rendered token ids (all train_on_eos modes, shared closing / opening
markers, longest-opening-marker rule), message normalisation with column images, user-declared boundaries, and the
collator around a stand-in processor."""
import pytest
import torch

from axolotl_b200.data.multimodal import (MultiModalChatCollator, ProcessingStrategy, RoleBoundary, family_boundaries,
                                          get_processing_strategy, normalize_example, resolve_role_boundaries,
                                          role_keep_mask)


class Tok:
    """Whitespace tokenizer with a growing vocabulary; special markers are single tokens."""
    SPECIAL = ["<|im_start|>", "<|im_end|>", "<|image_pad|>", "[INST]", "[/INST]", "</s>", "<pad>", "\n",
               "<start_of_turn>", "<end_of_turn>"]

    def __init__(self):
        self.vocab = {t: i for i, t in enumerate(self.SPECIAL)}
        self.eos_token_id, self.pad_token_id, self.unk_token_id = self.vocab["</s>"], self.vocab["<pad>"], None
        self.chat_template = None

    def _split(self, text):
        out, cur = [], ""
        i = 0
        while i < len(text):
            for sp in self.SPECIAL:
                if text.startswith(sp, i):
                    if cur.strip():
                        out += cur.split()
                    cur = ""
                    out.append(sp)
                    i += len(sp)
                    break
            else:
                cur += text[i]
                i += 1
        if cur.strip():
            out += cur.split()
        return out

    def encode(self, text, add_special_tokens=False):
        return [self.vocab.setdefault(t, len(self.vocab)) for t in self._split(text)]

    def convert_tokens_to_ids(self, t):
        return self.vocab.get(t, self.unk_token_id)


def chatml(tok, turns):
    text = "".join(f"<|im_start|>{r}\n{c}<|im_end|>\n" for r, c in turns)
    return tok.encode(text)


def kept(tok, ids, mask):
    inv = {i: t for t, i in tok.vocab.items()}
    return [inv[i] for i, m in zip(ids, mask.tolist()) if m]


def test_role_mask_chatml_modes():
    tok = Tok()
    b = family_boundaries("qwen2_vl", tok)
    assert [x.role for x in b] == ["system", "user", "assistant"]
    ids = chatml(tok, [("system", "be brief"), ("user", "hi <|image_pad|> there"), ("assistant", "hello you"),
                       ("user", "more"), ("assistant", "sure thing")])
    m = role_keep_mask([ids], b, ["assistant"], "turn")[0]
    assert kept(tok, ids, m) == ["hello", "you", "<|im_end|>", "sure", "thing", "<|im_end|>"]
    m = role_keep_mask([ids], b, ["assistant"], "none")[0]
    assert kept(tok, ids, m) == ["hello", "you", "sure", "thing"]
    m = role_keep_mask([ids], b, ["assistant"], "last")[0]
    assert kept(tok, ids, m) == ["hello", "you", "sure", "thing", "<|im_end|>"]
    m = role_keep_mask([ids], b, ["assistant"], "all")[0]
    assert kept(tok, ids, m).count("<|im_end|>") == 5 and "hi" not in kept(tok, ids, m)
    m = role_keep_mask([ids], b, ["assistant", "user"], "turn")[0]
    assert kept(tok, ids, m)[:4] == ["hi", "<|image_pad|>", "there", "<|im_end|>"]
    assert not role_keep_mask([ids], b, [], "turn").any()
    with pytest.raises(ValueError):
        role_keep_mask([ids], b, ["assistant"], "sometimes")


def test_shared_closing_marker_is_rescanned_as_the_next_opening():
    tok = Tok()
    b = family_boundaries("pixtral", tok)
    ids = tok.encode("[INST] what is this [/INST] a cat </s> [INST] sure ? [/INST] yes </s>")
    m = role_keep_mask([ids], b, ["assistant"], "turn")[0]
    assert kept(tok, ids, m) == ["a", "cat", "</s>", "yes", "</s>"]
    # "all" must not leak the user's [/INST]: it is not part of the user turn
    m = role_keep_mask([ids], b, ["assistant"], "all")[0]
    assert "[/INST]" not in kept(tok, ids, m)


def test_longest_opening_marker_wins_and_unterminated_turn_runs_to_the_end():
    tok = Tok()
    short = RoleBoundary("user", tok.encode("<|im_start|>"), tok.encode("<|im_end|>"))
    long_ = RoleBoundary("assistant", tok.encode("<|im_start|>assistant\n"), tok.encode("<|im_end|>"))
    ids = tok.encode("<|im_start|>assistant\nfine and more")
    m = role_keep_mask([ids], [short, long_], ["assistant"], "turn")[0]
    assert kept(tok, ids, m) == ["fine", "and", "more"]
    inc = RoleBoundary("assistant", tok.encode("<|im_start|>assistant\n"), tok.encode("<|im_end|>"), include_start=True)
    m = role_keep_mask([ids], [inc], ["assistant"], "turn")[0]
    assert kept(tok, ids, m)[0] == "<|im_start|>"


def test_user_declared_boundaries_and_their_errors():
    tok = Tok()
    b = resolve_role_boundaries([{"role": "assistant", "start": "<start_of_turn>model\n", "end": "<end_of_turn>"},
                                 {"role": "user", "start": "<start_of_turn>user\n", "end": "eos_token"},
                                 {"role": "tool", "start": "[INST]"}], tok)
    assert b[1].end_tokens == [tok.eos_token_id] and b[2].end_tokens == []
    with pytest.raises(ValueError, match="role"):
        resolve_role_boundaries([{"start": "x"}], tok)
    with pytest.raises(ValueError, match="tokenises to nothing"):
        resolve_role_boundaries([{"role": "a", "start": "   "}], tok)


def test_normalize_example_schemas_and_column_image():
    ex = {"conversations": [{"from": "human", "value": "look"}, {"from": "gpt", "value": "ok"}], "images": ["not-a-file"]}
    out = normalize_example(ex)
    assert [m["role"] for m in out["messages"]] == ["user", "assistant"] and "conversations" not in out
    assert out["messages"][0]["content"][-1] == {"type": "image", "image": "not-a-file"}
    assert ex["conversations"][0]["value"] == "look"                       # the input row is untouched
    ex = {"chat": [{"role": "user", "content": [{"type": "image"}, {"type": "text", "text": "what?"}]},
                   {"role": "assistant", "content": "a dog", "weight": None}], "image": "img0"}
    out = normalize_example(ex, field_messages="chat")
    assert out["messages"][0]["content"][0] == {"type": "image", "image": "img0"}      # the bare placeholder is filled
    assert out["messages"][1] == {"role": "assistant", "content": [{"type": "text", "text": "a dog"}]}
    with pytest.raises(ValueError):
        normalize_example({"text": "x"})
    with pytest.raises(ValueError):
        normalize_example({"messages": None})


class Processor:
    image_token = "<|image_pad|>"

    def __init__(self):
        self.tokenizer = Tok()

    def apply_chat_template(self, conversations, add_generation_prompt=False, tokenize=True, return_tensors="pt",
                            return_dict=True, chat_template=None, processor_kwargs=None):
        rows = []
        for msgs in conversations:
            text = ""
            for m in msgs:
                body = " ".join("<|image_pad|> <|image_pad|>" if p["type"] == "image" else p["text"] for p in m["content"])
                text += f"<|im_start|>{m['role']}\n{body}<|im_end|>\n"
            rows.append(self.tokenizer.encode(text))
        L = max(len(r) for r in rows)
        ids = torch.tensor([r + [self.tokenizer.pad_token_id] * (L - len(r)) for r in rows])
        return {"input_ids": ids, "attention_mask": (ids != self.tokenizer.pad_token_id).long(),
                "pixel_values": torch.zeros(len(rows), 3, 4, 4)}


def test_collator_masks_roles_pad_and_media_tokens():
    proc = Processor()
    strat = get_processing_strategy(proc, chat_template_type="qwen2_vl")
    coll = MultiModalChatCollator(proc.tokenizer, strat)
    batch = coll([
        {"messages": [{"role": "user", "content": "describe"}, {"role": "assistant", "content": "a red square"}], "images": ["i"]},
        {"messages": [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "yo"}]},
    ])
    ids, labels = batch["input_ids"], batch["labels"]
    assert labels.shape == ids.shape and "pixel_values" in batch
    tok = proc.tokenizer
    for r in range(2):
        words = kept(tok, ids[r].tolist(), labels[r] != -100)
        assert words == (["a", "red", "square", "<|im_end|>"] if r == 0 else ["yo", "<|im_end|>"])
    assert (labels[ids == tok.vocab["<|image_pad|>"]] == -100).all() and (labels[ids == tok.pad_token_id] == -100).all()
    # train_on_inputs keeps everything except pad and media tokens
    strat2 = ProcessingStrategy(proc, family="qwen2_vl", train_on_inputs=True)
    lab2 = strat2.process_labels(ids)
    assert (lab2 != -100).sum() == ((ids != tok.pad_token_id) & (ids != tok.vocab["<|image_pad|>"])).sum()
    with pytest.raises(ValueError):
        MultiModalChatCollator(tok, strat, packing=True)
    # a family without token-level role markers masks only pad / media tokens
    strat3 = get_processing_strategy(proc, chat_template_type="glm4v")
    assert strat3.boundaries == [] and (strat3.process_labels(ids) != -100).sum() == (lab2 != -100).sum()
