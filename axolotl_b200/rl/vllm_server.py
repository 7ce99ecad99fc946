"""Generation server for online RL: a thin FastAPI front on a vLLM engine (library code, run as a
separate process by ``axolotl vllm-serve CONFIG``). Protocol used by rl.grpo.VLLMServerRollout:

* ``GET  /health/``                                   -> {"status": "ok"}
* ``POST /generate/``  {prompt_ids, n, max_tokens, temperature, top_p, top_k} -> {"completion_ids": [...]}
* ``POST /load_adapter/`` {path, step}                -> subsequent generations use that LoRA adapter

Reference: src/axolotl/cli/vllm_serve.py and src/axolotl/scripts/vllm_serve_lora.py (a trl
``vllm_serve`` wrapper with LoRA-file synchronisation).
"""
from __future__ import annotations


def build_app(llm, sampling_cls, lora_request_cls):
    from fastapi import FastAPI
    from pydantic import BaseModel

    app = FastAPI()
    state = {"lora": None, "step": 0}

    class GenerateRequest(BaseModel):
        prompt_ids: list[list[int]]
        n: int = 1
        max_tokens: int = 256
        temperature: float = 1.0
        top_p: float = 1.0
        top_k: int = -1

    class AdapterRequest(BaseModel):
        path: str
        step: int = 0

    @app.get("/health/")
    def health():
        return {"status": "ok", "adapter_step": state["step"]}

    @app.post("/generate/")
    def generate(req: GenerateRequest):
        sp = sampling_cls(n=req.n, max_tokens=req.max_tokens, temperature=req.temperature, top_p=req.top_p,
                          top_k=req.top_k)
        outs = llm.generate([{"prompt_token_ids": p} for p in req.prompt_ids], sampling_params=sp,
                            lora_request=state["lora"], use_tqdm=False)
        return {"completion_ids": [list(c.token_ids) for o in outs for c in o.outputs]}

    @app.post("/load_adapter/")
    def load_adapter(req: AdapterRequest):
        state["step"] = req.step
        # a new integer id per step makes the engine reload the files instead of reusing its cache
        state["lora"] = lora_request_cls(f"policy-{req.step}", req.step + 1, req.path)
        return {"status": "ok"}

    return app


def serve(cfg):
    try:
        from vllm import LLM, SamplingParams
        from vllm.lora.request import LoRARequest
    except ImportError as exc:   # pragma: no cover - depends on the environment
        raise RuntimeError("vllm-serve needs the vllm package") from exc
    import uvicorn

    v = dict(cfg.get("vllm") or {})
    t = dict(cfg.get("trl") or {})
    llm = LLM(model=cfg["base_model"], tensor_parallel_size=v.get("tensor_parallel_size") or 1,
              gpu_memory_utilization=v.get("gpu_memory_utilization") or 0.9, dtype=v.get("dtype") or "auto",
              max_model_len=v.get("max_model_len"), enable_lora=bool(cfg.get("adapter")),
              max_lora_rank=max(cfg.get("lora_r") or 16, 8), enable_prefix_caching=v.get("enable_prefix_caching"))
    app = build_app(llm, SamplingParams, LoRARequest)
    uvicorn.run(app, host=v.get("host") or t.get("vllm_server_host") or "0.0.0.0",
                port=int(v.get("port") or t.get("vllm_server_port") or 8000))
