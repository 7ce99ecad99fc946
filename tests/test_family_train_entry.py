"""The training entry point (config validation -> architecture descriptor -> model build -> adapter -> trainer) on a
small random checkpoint of the newer model families: the path a user takes, not just the model graph."""
import pytest
import torch

from axolotl_b200.config.load import load_cfg
from axolotl_b200.io import hf as hf_io
from axolotl_b200.models.config import ModelConfig
from axolotl_b200.models.transformer import CausalLM
from axolotl_b200.train.run import train

@pytest.fixture(autouse=True)
def _no_plugins_left_over():
    """Plugins are a process-wide registry; a run here must not inherit what an earlier test module registered."""
    from axolotl_b200.plugins.base import PluginManager

    PluginManager.reset()
    yield
    PluginManager.reset()


FAMILIES = {
    "gemma2": dict(model_type="gemma2", vocab_size=320, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                   num_attention_heads=4, num_key_value_heads=2, head_dim=16, query_pre_attn_scalar=16, sliding_window=32,
                   max_position_embeddings=256),
    "falcon_h1": dict(model_type="falcon_h1", vocab_size=320, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=16, mamba_d_ssm=96, mamba_n_heads=8, mamba_d_head=12,
                      mamba_n_groups=2, mamba_d_state=16, mamba_d_conv=4, mamba_chunk_size=8, mamba_rms_norm=True,
                      mamba_norm_before_gate=False, rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=256,
                      ssm_multipliers=[0.9, 1.1, 1.2, 0.8, 1.3], mlp_multipliers=[0.8, 1.4], key_multiplier=0.8),
    "glm_moe_dsa": dict(model_type="glm_moe_dsa", vocab_size=320, hidden_size=64, intermediate_size=96, moe_intermediate_size=32,
                        num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=4, n_routed_experts=4, n_shared_experts=1,
                        num_experts_per_tok=2, mlp_layer_types=["dense", "sparse"], q_lora_rank=24, kv_lora_rank=16,
                        qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=12, index_topk=12, index_head_dim=16, index_n_heads=4,
                        max_position_embeddings=256, tie_word_embeddings=False),
    "qwen3_next": dict(model_type="qwen3_next", vocab_size=320, hidden_size=64, intermediate_size=96, num_hidden_layers=4,
                       num_attention_heads=4, num_key_value_heads=2, head_dim=16, linear_num_value_heads=4, linear_num_key_heads=2,
                       linear_key_head_dim=8, linear_value_head_dim=8, linear_conv_kernel_dim=4, num_experts=4,
                       num_experts_per_tok=2, moe_intermediate_size=32, shared_expert_intermediate_size=32,
                       max_position_embeddings=256, tie_word_embeddings=False),
    "deepseek_v3": dict(model_type="deepseek_v3", vocab_size=320, hidden_size=64, intermediate_size=96, moe_intermediate_size=32,
                        num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=4, n_routed_experts=4, n_shared_experts=1,
                        num_experts_per_tok=2, n_group=2, topk_group=1, first_k_dense_replace=1, q_lora_rank=24, kv_lora_rank=16,
                        qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=12, max_position_embeddings=256,
                        tie_word_embeddings=False),
    "granitemoehybrid": dict(model_type="granitemoehybrid", vocab_size=320, hidden_size=64, intermediate_size=48,
                             shared_intermediate_size=96, num_hidden_layers=3, layer_types=["mamba", "attention", "mamba"],
                             num_attention_heads=4, num_key_value_heads=2, mamba_n_heads=8, mamba_d_head=16, mamba_n_groups=2,
                             mamba_d_state=16, mamba_d_conv=4, mamba_expand=2, mamba_chunk_size=8, num_local_experts=4,
                             num_experts_per_tok=2, position_embedding_type="nope", tie_word_embeddings=True,
                             embedding_multiplier=3.0, attention_multiplier=0.2, residual_multiplier=0.5, logits_scaling=2.0,
                             max_position_embeddings=256),
    "llama4_text": dict(model_type="llama4_text", vocab_size=320, hidden_size=64, intermediate_size=48, intermediate_size_mlp=96,
                        num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=16, num_local_experts=4,
                        num_experts_per_tok=1, interleave_moe_layer_step=2, no_rope_layers=[1, 1, 1, 0], attention_chunk_size=16,
                        floor_scale=8, attn_scale=0.1, tie_word_embeddings=False, max_position_embeddings=256,
                        layer_types=["chunked_attention", "chunked_attention", "chunked_attention", "full_attention"]),
    "nemotron_h": dict(model_type="nemotron_h", vocab_size=320, hidden_size=64, layers_block_type=["mamba", "attention", "mlp", "mamba"],
                       num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=96, mlp_hidden_act="relu2",
                       ssm_state_size=16, mamba_num_heads=8, mamba_head_dim=12, n_groups=2, conv_kernel=4, chunk_size=8,
                       tie_word_embeddings=False, max_position_embeddings=256),
    "glm4": dict(model_type="glm4", vocab_size=320, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                 num_key_value_heads=2, head_dim=16, partial_rotary_factor=0.5, attention_bias=True, tie_word_embeddings=False,
                 max_position_embeddings=256),
    "olmo3": dict(model_type="olmo3", vocab_size=320, hidden_size=64, intermediate_size=96, num_hidden_layers=4,
                  num_attention_heads=4, num_key_value_heads=2, tie_word_embeddings=False, max_position_embeddings=256,
                  sliding_window=8, layer_types=["sliding_attention", "sliding_attention", "sliding_attention", "full_attention"]),
    "arcee": dict(model_type="arcee", vocab_size=320, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                  num_attention_heads=4, num_key_value_heads=2, head_dim=16, hidden_act="relu2", tie_word_embeddings=False,
                  max_position_embeddings=256),
    "glm4_moe": dict(model_type="glm4_moe", vocab_size=320, hidden_size=64, intermediate_size=96, moe_intermediate_size=32,
                     num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16, n_routed_experts=4,
                     n_shared_experts=1, num_experts_per_tok=2, first_k_dense_replace=1, use_qk_norm=True, attention_bias=True,
                     tie_word_embeddings=False, max_position_embeddings=256),
    "granitemoeshared": dict(model_type="granitemoeshared", vocab_size=320, hidden_size=64, intermediate_size=48,
                             shared_intermediate_size=96, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                             num_local_experts=4, num_experts_per_tok=2, tie_word_embeddings=True, embedding_multiplier=3.0,
                             attention_multiplier=0.2, residual_multiplier=0.5, logits_scaling=2.0, max_position_embeddings=256),
    "hunyuan_v1_dense": dict(model_type="hunyuan_v1_dense", vocab_size=320, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                             num_attention_heads=4, num_key_value_heads=2, head_dim=16, tie_word_embeddings=False,
                             max_position_embeddings=256),
    "ernie4_5": dict(model_type="ernie4_5", vocab_size=320, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                     num_attention_heads=4, num_key_value_heads=2, head_dim=16, use_bias=True, tie_word_embeddings=False,
                     max_position_embeddings=256),
    "starcoder2": dict(model_type="starcoder2", vocab_size=320, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                       num_attention_heads=4, num_key_value_heads=2, use_bias=True, sliding_window=16, tie_word_embeddings=True,
                       max_position_embeddings=256),
    "cohere2": dict(model_type="cohere2", vocab_size=320, hidden_size=64, intermediate_size=96, num_hidden_layers=4,
                    num_attention_heads=4, num_key_value_heads=2, logit_scale=0.25, tie_word_embeddings=True,
                    max_position_embeddings=256, sliding_window=8,
                    layer_types=["sliding_attention", "sliding_attention", "sliding_attention", "full_attention"]),
    "nemotron": dict(model_type="nemotron", vocab_size=320, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                     num_attention_heads=4, num_key_value_heads=2, head_dim=16, tie_word_embeddings=False,
                     max_position_embeddings=256),
    "qwen3_5_moe_text": dict(model_type="qwen3_5_moe_text", vocab_size=320, hidden_size=64, intermediate_size=96, num_hidden_layers=4,
                             num_attention_heads=4, num_key_value_heads=2, head_dim=16, linear_num_value_heads=4,
                             linear_num_key_heads=2, linear_key_head_dim=8, linear_value_head_dim=8, linear_conv_kernel_dim=4,
                             num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, shared_expert_intermediate_size=32,
                             tie_word_embeddings=False, max_position_embeddings=256),
    "ministral3": dict(model_type="ministral3", vocab_size=320, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                       num_attention_heads=4, num_key_value_heads=2, head_dim=16, tie_word_embeddings=False,
                       max_position_embeddings=256),
    "hunyuan_v1_moe": dict(model_type="hunyuan_v1_moe", vocab_size=320, hidden_size=64, intermediate_size=48, num_hidden_layers=2,
                           num_attention_heads=4, num_key_value_heads=2, head_dim=16, num_experts=4, moe_topk=2,
                           tie_word_embeddings=False, max_position_embeddings=256),
    "ernie4_5_moe": dict(model_type="ernie4_5_moe", vocab_size=320, hidden_size=64, intermediate_size=96, moe_intermediate_size=32,
                         num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, moe_num_experts=4, moe_k=2,
                         moe_num_shared_experts=1, moe_layer_start_index=1, moe_layer_interval=1, moe_layer_end_index=-1,
                         tie_word_embeddings=False, max_position_embeddings=256),
    "apertus": dict(model_type="apertus", vocab_size=320, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                    num_attention_heads=4, num_key_value_heads=2, tie_word_embeddings=False, max_position_embeddings=256,
                    rope_parameters={"rope_type": "default", "rope_theta": 10000.0}),
    "minimax_m2": dict(model_type="minimax_m2", vocab_size=320, hidden_size=64, intermediate_size=32, num_hidden_layers=2,
                       num_attention_heads=4, num_key_value_heads=2, head_dim=16, num_local_experts=4, num_experts_per_tok=2,
                       tie_word_embeddings=False, max_position_embeddings=256),
    "lfm2": dict(model_type="lfm2", vocab_size=320, hidden_size=64, intermediate_size=96, num_hidden_layers=3, num_attention_heads=4,
                 num_key_value_heads=2, layer_types=["conv", "full_attention", "conv"], conv_L_cache=3,
                 block_auto_adjust_ff_dim=False, tie_word_embeddings=True, max_position_embeddings=256),
    "mistral4": dict(model_type="mistral4", vocab_size=320, hidden_size=64, intermediate_size=96, moe_intermediate_size=32,
                     num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=4, n_routed_experts=4, n_shared_experts=1,
                     num_experts_per_tok=2, first_k_dense_replace=1, q_lora_rank=24, kv_lora_rank=16, qk_nope_head_dim=8,
                     qk_rope_head_dim=8, v_head_dim=16, tie_word_embeddings=False, max_position_embeddings=256),
    "phi": dict(model_type="phi", vocab_size=320, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                num_key_value_heads=2, tie_word_embeddings=False, max_position_embeddings=256),
    "olmo": dict(model_type="olmo", vocab_size=320, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                 num_key_value_heads=2, clip_qkv=8.0, tie_word_embeddings=False, max_position_embeddings=256),
    "lfm2_moe": dict(model_type="lfm2_moe", vocab_size=320, hidden_size=64, intermediate_size=96, moe_intermediate_size=32,
                     num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2, layer_types=["conv", "full_attention", "conv"],
                     conv_L_cache=3, num_experts=4, num_experts_per_tok=2, num_dense_layers=1, tie_word_embeddings=True,
                     max_position_embeddings=256),
    "afmoe": dict(model_type="afmoe", vocab_size=320, hidden_size=64, intermediate_size=96, moe_intermediate_size=32, num_hidden_layers=4,
                  num_attention_heads=4, num_key_value_heads=2, head_dim=16, num_experts=4, num_experts_per_tok=2, num_shared_experts=1,
                  num_dense_layers=1, sliding_window=32, tie_word_embeddings=False, max_position_embeddings=256),
    "gemma4_text": dict(model_type="gemma4_text", vocab_size=320, hidden_size=64, intermediate_size=96, num_hidden_layers=3,
                        num_attention_heads=4, num_key_value_heads=2, head_dim=16, global_head_dim=32, sliding_window=16,
                        layer_types=["sliding_attention", "sliding_attention", "full_attention"], hidden_size_per_layer_input=0,
                        attention_k_eq_v=True, num_global_key_value_heads=1, tie_word_embeddings=True, max_position_embeddings=256),
    "gemma4_text_full": dict(model_type="gemma4_text", vocab_size=320, hidden_size=64, intermediate_size=96, num_hidden_layers=4,
                             num_attention_heads=4, num_key_value_heads=2, head_dim=16, global_head_dim=32, sliding_window=16,
                             layer_types=["sliding_attention", "full_attention", "sliding_attention", "full_attention"],
                             hidden_size_per_layer_input=16, vocab_size_per_layer_input=320, num_kv_shared_layers=2,
                             enable_moe_block=True, num_experts=4, top_k_experts=2, moe_intermediate_size=32,
                             tie_word_embeddings=True, max_position_embeddings=256),
    "falcon": dict(model_type="falcon", vocab_size=320, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_kv_heads=2,
                   new_decoder_architecture=True, ffn_hidden_size=160, max_position_embeddings=256, tie_word_embeddings=True),
    "gpt_oss": dict(model_type="gpt_oss", vocab_size=320, hidden_size=64, intermediate_size=48, num_hidden_layers=2,
                    num_attention_heads=4, num_key_value_heads=2, head_dim=16, num_local_experts=4, num_experts_per_tok=2,
                    sliding_window=8, layer_types=["sliding_attention", "full_attention"], tie_word_embeddings=False,
                    max_position_embeddings=256, attention_bias=True, swiglu_limit=7.0),
}


@pytest.mark.parametrize("family", sorted(FAMILIES))
def test_lora_training_run_from_a_checkpoint_directory(tmp_path, family):
    mc = ModelConfig.from_hf_dict(FAMILIES[family])
    hf_io.save_pretrained(CausalLM(mc, dtype=torch.float32).init_weights(1), str(tmp_path / "base"))
    cfg = load_cfg({"base_model": str(tmp_path / "base"), "adapter": "lora", "lora_r": 4, "lora_alpha": 8, "lora_target_linear": True,
                    "sequence_len": 128, "micro_batch_size": 1, "gradient_accumulation_steps": 1, "max_steps": 3,
                    "learning_rate": 2e-3, "lr_scheduler": "constant", "output_dir": str(tmp_path / "out"), "device": "cpu",
                    "sample_packing": True, "save_strategy": "no", "logging_steps": 1,
                    "datasets": [{"path": "synthetic", "type": "_synthetic", "length": 12, "min_length": 20, "max_length": 60,
                                  "max_input_id": 300}]})
    model, _, trainer = train(cfg)
    assert trainer.global_step == 3
    losses = [h["loss"] for h in trainer.log_history if "loss" in h]
    assert all(l == l and l < 20 for l in losses), losses          # finite
    trained = [n for n, p in model.named_parameters() if p.requires_grad]
    assert trained and all("lora" in n for n in trained), trained[:5]


@pytest.mark.parametrize("family", sorted(FAMILIES))
def test_adapter_save_and_sharded_merge_reproduce_the_adapted_model(tmp_path, family):
    """adapter_model.safetensors in the checkpoint's own tensor names -> shard-by-shard merge -> same logits."""
    from axolotl_b200.io.merge import merge_lora_sharded
    from axolotl_b200.models.lora import LoraSpec, discover_linear_names, inject_lora, save_adapter

    mc = ModelConfig.from_hf_dict(FAMILIES[family])
    model = CausalLM(mc, dtype=torch.float32).init_weights(2)
    hf_io.save_pretrained(model, str(tmp_path / "base"))
    names = discover_linear_names(model)
    assert "o_proj" in names and "weights_proj" not in names
    spec = LoraSpec(r=4, lora_alpha=8, target_modules=names)
    inject_lora(model, spec)
    g = torch.Generator().manual_seed(5)
    with torch.no_grad():
        for n, p in model.named_parameters():
            if "lora_B" in n:
                p.copy_(torch.randn(p.shape, generator=g) * 0.05)
        for _, m in model.fused_linears():
            if getattr(m, "lora_B", None) is not None:          # keep the block-diagonal structure of fused projections
                keep = torch.zeros_like(m.lora_B)
                for (r0, rows, c0, r) in m.lora_blocks:
                    keep[r0:r0 + rows, c0:c0 + r] = 1
                m.lora_B.mul_(keep)
    save_adapter(model, spec, str(tmp_path / "ad"))
    ids = torch.randint(3, 300, (1, 40))
    model.eval()
    with torch.no_grad():
        want = model(ids, return_logits=True).logits
    res = merge_lora_sharded(str(tmp_path / "base"), str(tmp_path / "ad"), str(tmp_path / "merged"))
    assert res["unmatched"] == [], res["unmatched"][:5]
    merged = hf_io.load_pretrained(str(tmp_path / "merged"), dtype=torch.float32).eval()
    with torch.no_grad():
        got = merged(ids, return_logits=True).logits
    assert torch.allclose(got, want, atol=2e-4, rtol=1e-3), (got - want).abs().max()
