"""Image front ends: LLaVA (CLIP vision transformer + two-layer projector) and Gemma 3 (SigLIP vision transformer +
pooling projector), and the merge of the projected patch features into the language model's token embeddings.

A LLaVA checkpoint is three parts: ``vision_tower`` (CLIP ViT: patch convolution, class token, learned positions, pre-norm
encoder layers with biased projections and quick-GELU), ``multi_modal_projector`` (linear, GELU, linear) and
``language_model`` (one of the causal graphs of this package). The conversation's ``<image>`` placeholder tokens, one per
patch, are replaced by the projected features of the hidden state ``vision_feature_layer`` (default: the one before the
last layer) without its class token. The language model then runs unchanged: causal attention over text and image
positions alike, so packing, the fused loss and the adapters apply as they do for text.

The tower runs per image batch through library attention (bidirectional, 577 tokens per image for ViT-L/14 at 336 px: a
few percent of a step next to the language model). It is frozen unless the config says ``freeze_mm_modules: false``; the
projector trains in full fine-tuning and follows the adapter's freezing otherwise.

Gemma 3 checkpoints (``Gemma3ForConditionalGeneration``) differ in three ways: the tower is SigLIP (no class token, biased
patch convolution, tanh-GELU, the post-norm output is the feature), the projector average-pools the 64 x 64 patch grid to
``mm_tokens_per_image`` (256) soft tokens, RMS-normalises them and multiplies by one matrix, and the tokens of one image
attend each other in both directions inside the language model (``image_groups`` below; the attention then runs the
blocked library path, since the causal kernels cannot express it).

Behaviour of the reference's multimodal path on HF ``LlavaForConditionalGeneration`` / ``Gemma3ForConditionalGeneration``
(src/axolotl/loaders/constants.py:1-40 model mapping, src/axolotl/processing_strategies.py:46-1540 data side,
src/axolotl/utils/collators/mm_chat.py:15-59).
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

VISION_WRAPPERS = ("llava", "gemma3")


def _act(name):
    return {"quick_gelu": lambda x: x * torch.sigmoid(1.702 * x), "gelu": F.gelu,
            "gelu_pytorch_tanh": lambda x: F.gelu(x, approximate="tanh")}[name]


class _ClipAttention(nn.Module):
    def __init__(self, H, heads, dtype, device):
        super().__init__()
        self.heads = heads
        self.q_proj = nn.Linear(H, H, dtype=dtype, device=device)
        self.k_proj = nn.Linear(H, H, dtype=dtype, device=device)
        self.v_proj = nn.Linear(H, H, dtype=dtype, device=device)
        self.out_proj = nn.Linear(H, H, dtype=dtype, device=device)

    def forward(self, x):
        B, N, H = x.shape
        q, k, v = (p(x).view(B, N, self.heads, H // self.heads).transpose(1, 2) for p in (self.q_proj, self.k_proj, self.v_proj))
        return self.out_proj(F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B, N, H))


class _ClipMLP(nn.Module):
    def __init__(self, H, inter, act, dtype, device):
        super().__init__()
        self.fc1 = nn.Linear(H, inter, dtype=dtype, device=device)
        self.fc2 = nn.Linear(inter, H, dtype=dtype, device=device)
        self.act = _act(act)

    def forward(self, x):
        return self.fc2(self.act(self.fc1(x)))


class _ClipLayer(nn.Module):
    def __init__(self, H, heads, inter, act, eps, dtype, device):
        super().__init__()
        self.layer_norm1 = nn.LayerNorm(H, eps=eps, dtype=dtype, device=device)
        self.self_attn = _ClipAttention(H, heads, dtype, device)
        self.layer_norm2 = nn.LayerNorm(H, eps=eps, dtype=dtype, device=device)
        self.mlp = _ClipMLP(H, inter, act, dtype, device)

    def forward(self, x):
        x = x + self.self_attn(self.layer_norm1(x))
        return x + self.mlp(self.layer_norm2(x))


class _ClipEmbeddings(nn.Module):
    def __init__(self, H, image_size, patch, channels, dtype, device):
        super().__init__()
        self.class_embedding = nn.Parameter(torch.zeros(H, dtype=dtype, device=device))
        self.patch_embedding = nn.Conv2d(channels, H, kernel_size=patch, stride=patch, bias=False, dtype=dtype, device=device)
        self.num_positions = (image_size // patch) ** 2 + 1
        self.position_embedding = nn.Embedding(self.num_positions, H, dtype=dtype, device=device)

    def forward(self, pixel_values):
        p = self.patch_embedding(pixel_values.to(self.patch_embedding.weight.dtype)).flatten(2).transpose(1, 2)     # [B, N, H]
        if p.shape[1] + 1 != self.num_positions:
            raise ValueError(f"image gives {p.shape[1]} patches, the tower's position table has {self.num_positions - 1}")
        cls = self.class_embedding.expand(p.shape[0], 1, -1)
        return torch.cat([cls, p], 1) + self.position_embedding.weight[None]


class _ClipEncoder(nn.Module):
    def __init__(self, layers):
        super().__init__()
        self.layers = nn.ModuleList(layers)


class _ClipVisionModel(nn.Module):
    """Module tree under ``vision_tower.vision_model`` of the checkpoint (its names, misspelt ``pre_layrnorm`` included)."""

    def __init__(self, vc: dict, dtype, device):
        super().__init__()
        H, eps = int(vc["hidden_size"]), float(vc.get("layer_norm_eps", 1e-5))
        self.embeddings = _ClipEmbeddings(H, int(vc["image_size"]), int(vc["patch_size"]), int(vc.get("num_channels", 3)), dtype, device)
        self.pre_layrnorm = nn.LayerNorm(H, eps=eps, dtype=dtype, device=device)
        self.encoder = _ClipEncoder([_ClipLayer(H, int(vc["num_attention_heads"]), int(vc["intermediate_size"]),
                                                vc.get("hidden_act", "quick_gelu"), eps, dtype, device)
                                     for _ in range(int(vc["num_hidden_layers"]))])
        self.post_layernorm = nn.LayerNorm(H, eps=eps, dtype=dtype, device=device)

    def hidden_state(self, pixel_values, index: int):
        """``hidden_states[index]`` in the HF numbering: 0 = after the pre-norm, i = after layer i."""
        n = len(self.encoder.layers)
        stop = index if index >= 0 else n + 1 + index
        x = self.pre_layrnorm(self.embeddings(pixel_values))
        for layer in self.encoder.layers[:stop]:
            x = layer(x)
        return x


class ClipVisionTower(nn.Module):
    def __init__(self, vc: dict, dtype, device):
        super().__init__()
        if vc.get("model_type", "clip_vision_model") != "clip_vision_model":
            raise ValueError(f"vision tower '{vc.get('model_type')}' is not built; the CLIP vision transformer is")
        self.vision_model = _ClipVisionModel(vc, dtype, device)


class _SiglipEmbeddings(nn.Module):
    def __init__(self, H, image_size, patch, channels, dtype, device):
        super().__init__()
        self.patch_embedding = nn.Conv2d(channels, H, kernel_size=patch, stride=patch, dtype=dtype, device=device)
        self.num_positions = (image_size // patch) ** 2
        self.position_embedding = nn.Embedding(self.num_positions, H, dtype=dtype, device=device)

    def forward(self, pixel_values):
        p = self.patch_embedding(pixel_values.to(self.patch_embedding.weight.dtype)).flatten(2).transpose(1, 2)
        if p.shape[1] != self.num_positions:
            raise ValueError(f"image gives {p.shape[1]} patches, the tower's position table has {self.num_positions}")
        return p + self.position_embedding.weight[None]


class _SiglipVisionModel(nn.Module):
    """Module tree under ``vision_tower.vision_model`` of a SigLIP checkpoint (without its pooling head)."""

    def __init__(self, vc: dict, dtype, device):
        super().__init__()
        H, eps = int(vc["hidden_size"]), float(vc.get("layer_norm_eps", 1e-6))
        self.embeddings = _SiglipEmbeddings(H, int(vc["image_size"]), int(vc["patch_size"]), int(vc.get("num_channels", 3)), dtype, device)
        self.encoder = _ClipEncoder([_ClipLayer(H, int(vc["num_attention_heads"]), int(vc["intermediate_size"]),
                                                vc.get("hidden_act", "gelu_pytorch_tanh"), eps, dtype, device)
                                     for _ in range(int(vc["num_hidden_layers"]))])
        self.post_layernorm = nn.LayerNorm(H, eps=eps, dtype=dtype, device=device)

    def last_hidden_state(self, pixel_values):
        x = self.embeddings(pixel_values)
        for layer in self.encoder.layers:
            x = layer(x)
        return self.post_layernorm(x)


class SiglipVisionTower(nn.Module):
    def __init__(self, vc: dict, dtype, device):
        super().__init__()
        self.vision_model = _SiglipVisionModel(vc, dtype, device)


class _OnePlusRMSNorm(nn.Module):
    def __init__(self, dim, eps, dtype, device):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.zeros(dim, dtype=dtype, device=device))

    def forward(self, x):
        xf = x.float()
        xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)
        return (xf * (1.0 + self.weight.float())).to(x.dtype)


class Gemma3Projector(nn.Module):
    """Average-pool the patch grid to ``tokens_per_side`` squared soft tokens, RMS-normalise, project."""

    def __init__(self, vc: dict, text_hidden, mm_tokens, dtype, device):
        super().__init__()
        Hv = int(vc["hidden_size"])
        self.mm_input_projection_weight = nn.Parameter(torch.zeros(Hv, text_hidden, dtype=dtype, device=device))
        self.mm_soft_emb_norm = _OnePlusRMSNorm(Hv, float(vc.get("layer_norm_eps", 1e-6)), dtype, device)
        self.side = int(vc["image_size"]) // int(vc["patch_size"])
        self.kernel = self.side // int(mm_tokens ** 0.5)

    def forward(self, x):
        B, _, Hv = x.shape
        g = x.transpose(1, 2).reshape(B, Hv, self.side, self.side)
        g = F.avg_pool2d(g, self.kernel, self.kernel).flatten(2).transpose(1, 2)
        return self.mm_soft_emb_norm(g) @ self.mm_input_projection_weight


class LlavaProjector(nn.Module):
    def __init__(self, in_dim, out_dim, act, bias, dtype, device):
        super().__init__()
        self.linear_1 = nn.Linear(in_dim, out_dim, bias=bias, dtype=dtype, device=device)
        self.linear_2 = nn.Linear(out_dim, out_dim, bias=bias, dtype=dtype, device=device)
        self.act = _act(act)

    def forward(self, x):
        return self.linear_2(self.act(self.linear_1(x)))


class VisionFrontEnd(nn.Module):
    """``vision_tower`` + ``multi_modal_projector``; ``forward(pixel_values)`` -> [images * patches, text hidden]."""

    def __init__(self, wrapper: dict, text_hidden: int, dtype=torch.bfloat16, device=None):
        super().__init__()
        vc = dict(wrapper["vision_config"])
        self.image_token_id = int(wrapper["image_token_id"])
        self.kind = wrapper.get("model_type", "llava")
        self.bidirectional_images = self.kind == "gemma3"      # the tokens of one image see each other in both directions
        if self.kind == "gemma3":
            self.tokens_per_image = int(wrapper.get("mm_tokens_per_image", 256))
            self.vision_tower = SiglipVisionTower(vc, dtype, device)
            self.multi_modal_projector = Gemma3Projector(vc, text_hidden, self.tokens_per_image, dtype, device)
        else:
            layer = wrapper.get("vision_feature_layer", -2)
            if not isinstance(layer, int):
                raise ValueError("a list of vision feature layers is not supported; one layer index is")
            self.feature_layer = layer
            self.drop_class_token = wrapper.get("vision_feature_select_strategy", "default") == "default"
            self.tokens_per_image = (int(vc["image_size"]) // int(vc["patch_size"])) ** 2 + (0 if self.drop_class_token else 1)
            self.vision_tower = ClipVisionTower(vc, dtype, device)
            self.multi_modal_projector = LlavaProjector(int(vc["hidden_size"]), text_hidden, wrapper.get("projector_hidden_act", "gelu"),
                                                        bool(wrapper.get("multimodal_projector_bias", True)), dtype, device)
        for p in self.vision_tower.parameters():
            p.requires_grad_(False)

    def init_weights(self, std=0.02, seed=0):
        gen = torch.Generator(device=next(self.multi_modal_projector.parameters()).device)
        gen.manual_seed(seed + 1000)
        with torch.no_grad():
            for name, p in self.named_parameters():
                if p.dim() >= 2 or name.endswith(("class_embedding",)):
                    p.normal_(0.0, std, generator=gen)
                elif name.endswith("bias") or name.endswith("mm_soft_emb_norm.weight"):
                    p.zero_()
                else:
                    p.fill_(1.0)
        return self

    def forward(self, pixel_values):
        tower_trains = any(p.requires_grad for p in self.vision_tower.parameters())
        pixel_values = pixel_values.to(next(self.multi_modal_projector.parameters()).device)
        with torch.set_grad_enabled(tower_trains and torch.is_grad_enabled()):
            if self.kind == "gemma3":
                x = self.vision_tower.vision_model.last_hidden_state(pixel_values)
            else:
                x = self.vision_tower.vision_model.hidden_state(pixel_values, self.feature_layer)
                if self.drop_class_token:
                    x = x[:, 1:]
        x = self.multi_modal_projector(x)
        return x.reshape(-1, x.shape[-1])


def merge_image_features(h, ids, feats, image_token_id):
    """Rows of ``h`` [T, H] at the placeholder tokens become the image features, in order."""
    mask = ids == image_token_id
    n = int(mask.sum())
    if n != feats.shape[0]:
        raise ValueError(f"{n} image placeholder tokens in the batch, {feats.shape[0]} image features "
                         "(one placeholder per patch is expected; was the sequence truncated inside an image?)")
    return h.masked_scatter(mask[:, None], feats.to(h.dtype))


def image_groups(ids, image_token_id):
    """[T] int32: -1 for text, else the index of the run of placeholder tokens (one run per image) a position belongs to."""
    m = ids == image_token_id
    start = m & ~torch.cat([m.new_zeros(1), m[:-1]])
    return torch.where(m, start.cumsum(0) - 1, -1).to(torch.int32)
