"""Label masks of ``type: chat_template`` and the fixed-format strategies, on a word-level tokenizer whose
tokens can be read back as words (fixtures restated from the reference's tests/prompt_strategies/)."""
import pytest

tokenizers = pytest.importorskip("tokenizers")
from transformers import PreTrainedTokenizerFast  # noqa: E402

from axolotl_b200.data.chat_template import (ChatTemplateStrategy, convert_content_parts,  # noqa: E402
                                             template_message_variables)
from axolotl_b200.data.strategies import load_strategy  # noqa: E402
from axolotl_b200.data.tokenizer import CHAT_TEMPLATES  # noqa: E402

WORDS = ("<s> </s> <unk> <pad> <|im_start|> <|im_end|> <|eot|> system user assistant tool \n hello there how are you fine thanks "
         "be brief what is two plus four the answer [[dummy_message]] [[dummy_reasoning]] <think> </think> let me add them "
         "[INST] [/INST] <<SYS>> <</SYS>> <|system|> <|user|> <|model|> Persona: kind robot ### System: User: Response: "
         "Context: Question: Answer: sky blue why").split(" ")


def make_tok(template="chatml", isolate=r"\n|<\|[a-z_]+\|>|\[\[[a-z_]+\]\]|</?think>"):
    vocab = {w: i for i, w in enumerate(dict.fromkeys(WORDS))}
    t = tokenizers.Tokenizer(tokenizers.models.WordLevel(vocab, unk_token="<unk>"))
    # words and newlines are tokens of their own
    t.pre_tokenizer = tokenizers.pre_tokenizers.Sequence([
        tokenizers.pre_tokenizers.Split(tokenizers.Regex(isolate), "isolated"),
        tokenizers.pre_tokenizers.WhitespaceSplit()])
    tok = PreTrainedTokenizerFast(tokenizer_object=t, bos_token="<s>", eos_token="</s>", unk_token="<unk>", pad_token="<pad>")
    if template:
        tok.chat_template = CHAT_TEMPLATES[template]
    return tok


def words(tok, ids, labels):
    return [tok.convert_ids_to_tokens(i) for i, l in zip(ids, labels) if l != -100]


CONV = {"messages": [{"role": "system", "content": "be brief"}, {"role": "user", "content": "hello there"},
                     {"role": "assistant", "content": "how are you"}, {"role": "user", "content": "fine thanks"},
                     {"role": "assistant", "content": "the answer"}]}
CFG = {"sequence_len": 256, "eot_tokens": ["<|im_end|>"]}


def test_only_assistant_content_and_its_turn_terminator_are_trained():
    tok = make_tok()
    s = ChatTemplateStrategy(tok, CFG, {"type": "chat_template"})
    out = s.tokenize(CONV)
    assert words(tok, out["input_ids"], out["labels"]) == ["how", "are", "you", "<|im_end|>", "the", "answer", "<|im_end|>"]
    assert len(out["input_ids"]) == len(out["labels"]) == len(out["attention_mask"])
    # headers (role names, newlines) are never trained, not even for assistant turns
    assert "assistant" not in words(tok, out["input_ids"], out["labels"])


@pytest.mark.parametrize("opt,expect", [
    ("turn", ["how", "are", "you", "<|im_end|>", "the", "answer", "<|im_end|>"]),
    ("all", ["<|im_end|>", "<|im_end|>", "how", "are", "you", "<|im_end|>", "<|im_end|>", "the", "answer", "<|im_end|>"]),
    ("last", ["how", "are", "you", "the", "answer", "<|im_end|>"]),
    ("none", ["how", "are", "you", "the", "answer"]),
])
def test_train_on_eot_window(opt, expect):
    tok = make_tok()
    s = ChatTemplateStrategy(tok, CFG, {"type": "chat_template", "train_on_eot": opt, "train_on_eos": opt})
    out = s.tokenize(CONV)
    assert words(tok, out["input_ids"], out["labels"]) == expect


def test_roles_to_train_training_field_and_train_on_inputs():
    tok = make_tok()
    s = ChatTemplateStrategy(tok, CFG, {"type": "chat_template", "roles_to_train": ["user"], "train_on_eot": "none",
                                        "train_on_eos": "none"})
    out = s.tokenize(CONV)
    assert words(tok, out["input_ids"], out["labels"]) == ["hello", "there", "fine", "thanks"]
    row = {"messages": [dict(m) for m in CONV["messages"]]}
    row["messages"][2]["training"] = False        # first assistant turn explicitly masked
    row["messages"][1]["training"] = True         # a user turn explicitly trained
    s2 = ChatTemplateStrategy(tok, CFG, {"type": "chat_template", "train_on_eot": "none", "train_on_eos": "none"})
    out = s2.tokenize(row)
    assert words(tok, out["input_ids"], out["labels"]) == ["hello", "there", "the", "answer"]
    s3 = ChatTemplateStrategy(tok, dict(CFG, train_on_inputs=True), {"type": "chat_template", "train_on_eot": "none",
                                                                     "train_on_eos": "none"})
    out = s3.tokenize(CONV)
    assert words(tok, out["input_ids"], out["labels"]) == ["be", "brief", "hello", "there", "how", "are", "you", "fine", "thanks",
                                                           "the", "answer"]


def test_sharegpt_spelling_role_aliases_system_field_and_drop_system():
    tok = make_tok()
    row = {"system": "be brief", "conversations": [{"from": "human", "value": "hello there"}, {"from": "gpt", "value": "fine thanks"}]}
    s = ChatTemplateStrategy(tok, CFG, {"type": "chat_template", "field_messages": "conversations"})
    turns = s.conversation(row)
    assert [t["role"] for t in turns] == ["system", "user", "assistant"] and turns[0]["content"] == "be brief"
    out = s.tokenize(row)
    assert words(tok, out["input_ids"], out["labels"]) == ["fine", "thanks", "<|im_end|>"]
    s2 = ChatTemplateStrategy(tok, CFG, {"type": "chat_template", "field_messages": "conversations", "drop_system_message": True})
    assert [t["role"] for t in s2.conversation(row)] == ["user", "assistant"]
    s3 = ChatTemplateStrategy(tok, CFG, {"type": "chat_template", "field_messages": "conversations",
                                         "roles": {"assistant": ["human"], "user": ["gpt"]}})
    assert [t["role"] for t in s3.conversation(row)][1:] == ["assistant", "user"]


def test_training_detail_offsets_and_content_parts():
    tok = make_tok()
    row = {"messages": [{"role": "user", "content": "what is two plus two"},
                        {"role": "assistant", "content": "let me add them the answer is four",
                         "training_detail": [{"begin_offset": 0, "end_offset": 14, "train": False},
                                             {"begin_offset": 16, "end_offset": 33, "train": True}]}]}
    s = ChatTemplateStrategy(tok, CFG, {"type": "chat_template", "train_on_eot": "none", "train_on_eos": "none"})
    out = s.tokenize(row)
    assert words(tok, out["input_ids"], out["labels"]) == ["the", "answer", "is", "four"]
    # the same through content parts with per-part flags
    text, details = convert_content_parts([{"text": "let me add them", "train": False}, {"text": " the answer is four", "weight": 1}])
    assert text == "let me add them the answer is four"
    assert details == [{"begin_offset": 0, "end_offset": 14, "train": False}, {"begin_offset": 15, "end_offset": 33, "train": True}]
    row2 = {"messages": [row["messages"][0], {"role": "assistant", "content": [{"text": "let me add them", "train": False},
                                                                              {"text": " the answer is four", "train": True}]}]}
    out2 = s.tokenize(row2)
    assert words(tok, out2["input_ids"], out2["labels"]) == ["the", "answer", "is", "four"]
    assert convert_content_parts("plain") is None
    assert convert_content_parts([{"text": "a"}, {"text": "b"}]) == ("ab", None)


def test_split_thinking_moves_reasoning_into_the_templates_key():
    tok = make_tok("qwen3")
    row = {"messages": [{"role": "user", "content": "what is two plus two"},
                        {"role": "assistant", "content": "<think> let me add them </think> the answer is four"}]}
    s = ChatTemplateStrategy(tok, CFG, {"type": "chat_template", "split_thinking": True, "train_on_eot": "none", "train_on_eos": "none"})
    turns = s.conversation(row)
    assert turns[1]["reasoning_content"] == "let me add them" and turns[1]["content"] == "the answer is four"
    out = s.tokenize(row)
    trained = words(tok, out["input_ids"], out["labels"])
    assert trained[-4:] == ["the", "answer", "is", "four"] and "<think>" in trained and "add" in trained


def test_template_message_variables():
    assert template_message_variables(CHAT_TEMPLATES["chatml"]) == {"role", "content"}
    v = template_message_variables(CHAT_TEMPLATES["qwen3"])
    assert {"role", "content", "reasoning_content", "tool_calls"} <= v
    t = "{% for m in messages[1:] %}{% set x = m %}{{ x.name }}{% if 'weight' in m %}{{ m['extra'] }}{% endif %}{% endfor %}{{ messages[0]['content'] }}"
    assert template_message_variables(t) == {"name", "weight", "extra", "content"}


def test_extra_message_keys_survive_only_if_the_template_reads_them():
    tok = make_tok("qwen3")
    s = ChatTemplateStrategy(tok, CFG, {"type": "chat_template"})
    m = s.transform_message({"role": "assistant", "content": "fine", "tool_calls": [{"function": {"name": "f", "arguments": '{"a": 1}'}}],
                             "private_note": "x"})
    assert "private_note" not in m and m["tool_calls"][0]["function"]["arguments"] == {"a": 1}
    with pytest.raises(ValueError, match="not valid JSON"):
        s.transform_message({"role": "assistant", "content": "x", "tool_calls": [{"function": {"name": "f", "arguments": "{bad"}}]})


def test_eot_validation():
    tok = make_tok()
    with pytest.raises(ValueError, match="Conflict between train_on_eos and train_on_eot"):
        ChatTemplateStrategy(tok, {"sequence_len": 64, "eot_tokens": ["</s>"]}, {"type": "chat_template", "train_on_eos": "all",
                                                                                 "train_on_eot": "turn"})
    with pytest.raises(ValueError, match="encoded as multiple tokens"):
        tok2 = make_tok(None)
        tok2.chat_template = "{% for m in messages %}{{ m['content'] + 'hello there' }}{% endfor %}"
        ChatTemplateStrategy(tok2, {"sequence_len": 64, "eot_tokens": ["hello there"]}, {"type": "chat_template"})


def test_every_bundled_template_locates_assistant_turns():
    msgs = {"messages": [{"role": "user", "content": "hello there"}, {"role": "assistant", "content": "fine thanks"}]}
    for name in CHAT_TEMPLATES.keys():
        # whatever markers a template glues to the content, the content words stay tokens of their own
        tok = make_tok(name, isolate=r"hello|there|fine|thanks|\[\[dummy_message\]\]")
        s = ChatTemplateStrategy(tok, {"sequence_len": 256}, {"type": "chat_template", "train_on_eos": "none", "train_on_eot": "none"})
        out = s.tokenize(msgs)
        trained = words(tok, out["input_ids"], out["labels"])
        assert trained[:2] == ["fine", "thanks"] or trained[-2:] == ["fine", "thanks"], (name, trained)
        assert "hello" not in trained, name


def test_fixed_format_strategies():
    tok = make_tok(None)
    cfg = {"sequence_len": 256}
    s = load_strategy("llama2_chat", tok, cfg, {})
    out = s.tokenize({"conversations": [{"from": "system", "value": "be brief"}, {"from": "human", "value": "hello there"},
                                        {"from": "gpt", "value": "fine thanks"}, {"from": "human", "value": "why"},
                                        {"from": "gpt", "value": "the answer"}]})
    assert words(tok, out["input_ids"], out["labels"]) == ["fine", "thanks", "</s>", "the", "answer", "</s>"]
    toks = tok.convert_ids_to_tokens(out["input_ids"])
    assert toks[:5] == ["<s>", "[INST]", "<<SYS>>", "be", "brief"] and toks.count("<<SYS>>") == 1 and toks.count("[INST]") == 2
    s = load_strategy("metharme", tok, cfg, {})
    out = s.tokenize({"prompt": "<|system|> be brief <|user|> hello there <|model|>", "generation": "fine thanks"})
    assert words(tok, out["input_ids"], out["labels"]) == ["fine", "thanks", "</s>", "</s>", "</s>"]
    s = load_strategy("pygmalion", tok, cfg, {})
    out = s.tokenize({"conversations": [{"role": "system", "value": "kind robot\n<START>"}, {"role": "human", "value": "hello there"},
                                        {"role": "bot", "value": "fine thanks"}]})
    assert words(tok, out["input_ids"], out["labels"]) == ["fine", "thanks", "</s>"]
    assert tok.convert_ids_to_tokens(out["input_ids"])[:3] == ["<s>", "<|system|>", "Persona:"]
    s = load_strategy("orcamini", tok, cfg, {})
    out = s.tokenize({"system_prompt": "be brief", "question": "why", "response": "the answer"})
    assert words(tok, out["input_ids"], out["labels"]) == ["the", "answer", "</s>"]
    s = load_strategy("context_qa.load_v2", tok, cfg, {})
    out = s.tokenize({"context": "the sky is blue", "question": "why", "answer": "blue"})
    assert words(tok, out["input_ids"], out["labels"]) == ["Answer:", "blue", "</s>"]
    for name in ("context_qa", "context_qa.load_404", "creative_acr", "creative_acr.load_critique", "creative_acr.load_revise",
                 "messages"):
        assert load_strategy(name, make_tok(), cfg, {}) is not None
