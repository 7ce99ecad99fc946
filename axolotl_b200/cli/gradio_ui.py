"""Browser front end for `axolotl inference --gradio`: one text box in, generated text out, streamed in pieces.

The model (and adapter) of the config is built once; every request applies the tokenizer's chat template (when it has
one and no `--prompter`-style raw mode is asked for), generates with sampling and yields the text generated so far
after every few tokens. `gradio` is an optional dependency. Reference: src/axolotl/cli/inference.py:159-281
(`do_inference_gradio`; config keys `gradio_title`, `gradio_share`, `gradio_server_name`, `gradio_server_port`,
`gradio_max_new_tokens`, `gradio_temperature`).
"""
from __future__ import annotations

import torch


def build_generator(cfg, model, tokenizer, device, piece: int = 8):
    """``fn(instruction) -> iterator of the text so far``; the function handed to the interface."""
    max_new = int(cfg.get("gradio_max_new_tokens") or 1024)
    temperature = float(cfg.get("gradio_temperature") if cfg.get("gradio_temperature") is not None else 0.9)
    has_template = bool(getattr(tokenizer, "chat_template", None)) and not cfg.get("gradio_raw_prompt")

    def generate(instruction):
        if not instruction:
            return
        text = instruction.strip()
        if has_template:
            ids = tokenizer.apply_chat_template([{"role": "user", "content": text}], add_generation_prompt=True, tokenize=True)
            ids = ids["input_ids"] if isinstance(ids, dict) else ids
        else:
            ids = tokenizer(text)["input_ids"]
        ids = torch.tensor([list(ids)], device=device)
        start, done = ids.shape[1], 0
        model.eval()
        with torch.no_grad():
            while done < max_new:
                n = min(piece, max_new - done)
                out = model.generate(ids, max_new_tokens=n, temperature=temperature, top_p=0.95, eos_token_id=tokenizer.eos_token_id)
                grew = out.shape[1] - ids.shape[1]
                ids, done = out, done + grew
                yield tokenizer.decode(ids[0, start:].tolist(), skip_special_tokens=True)
                if grew < n or (tokenizer.eos_token_id is not None and int(ids[0, -1]) == tokenizer.eos_token_id):
                    break
    return generate


def launch(cfg, gr=None):
    """Builds the model of ``cfg`` and serves the interface (blocks until the server stops)."""
    if gr is None:
        try:
            import gradio as gr
        except ImportError as e:
            raise RuntimeError("`axolotl inference --gradio` needs the `gradio` package, which is not installed") from e
    from ..data.tokenizer import load_tokenizer
    from ..train.evaluate import _device
    from ..train.run import build_model, setup_adapter

    dev = _device(cfg)
    tok = load_tokenizer(cfg)
    model = build_model(cfg, dev)
    setup_adapter(cfg, model)
    demo = gr.Interface(fn=build_generator(cfg, model, tok, dev), inputs="textbox", outputs="text",
                        title=cfg.get("gradio_title") or "Axolotl Gradio Interface")
    share = cfg.get("gradio_share")
    return demo.launch(share=True if share is None else bool(share), server_name=cfg.get("gradio_server_name") or "127.0.0.1",
                       server_port=cfg.get("gradio_server_port"))
