"""LongCat-Image transformer (vllm_omni/diffusion/models/longcat_image/longcat_image_transformer.py:
301-703): the FLUX layout (19 double-stream + 38 single-stream blocks, q/k RMSNorm, interleaved
3-axis rotary embedding, AdaLN-Zero) conditioned on the timestep only — no pooled text vector and
no guidance embedding — with position ids that carry a modality axis: text token i sits at
(0, i, i), image patch (y, x) at (1, y + 512, x + 512) (the offset is the tokenizer's maximum
length, pipeline_longcat_image.py:112-133,412-418).  Checkpoint names are FLUX's except
``time_embed.timestep_embedder``.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..flux.transformer import FluxTransformer2DModel, FluxTransformerConfig


@dataclass
class LongCatTransformerConfig(FluxTransformerConfig):
    joint_attention_dim: int = 3584
    pooled_projection_dim: int = 3584
    guidance_embeds: bool = False
    text_position_offset: int = 512


def longcat_rope_angles(h: int, w: int, txt_len: int, axes, offset: int, theta: float = 10000.0,
                        image_modality: int = 1, frames: int = 1) -> torch.Tensor:
    """Angles [frames*h*w + txt_len, sum(axes)/2]; image rows first, then text rows.  Text token i
    sits at (0, i, i), image patch (y, x) of frame f at (image_modality + f, y + offset, x + offset):
    the noise rows are modality 1, a conditioning image appended for editing is modality 2
    (pipeline_longcat_image_edit.py:456-470)."""
    def ang(idx, dim):
        inv = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float64) / dim))
        return torch.outer(idx.double(), inv).float()
    ys = torch.arange(h).repeat_interleave(w) + offset
    xs = torch.arange(w).repeat(h) + offset
    t = torch.arange(txt_len)
    img = torch.cat([torch.cat([ang(torch.full((h * w,), float(image_modality + f)), axes[0]), ang(ys, axes[1]),
                                ang(xs, axes[2])], dim=-1) for f in range(frames)], dim=0)
    txt = torch.cat([ang(torch.zeros(txt_len), axes[0]), ang(t, axes[1]), ang(t, axes[2])], dim=-1)
    return torch.cat([img, txt], dim=0)


class LongCatImageTransformer2DModel(FluxTransformer2DModel):
    def __init__(self, cfg: LongCatTransformerConfig | None = None, dtype=torch.bfloat16, device=None):
        cfg = cfg or LongCatTransformerConfig()
        cfg.guidance_embeds = False
        super().__init__(cfg, dtype=dtype, device=device)
        self.pooled_1 = self.pooled_2 = None            # conditioned on the timestep alone

    def _cos_sin(self, h, w, txt_len, device, frames: int = 1):
        key = (h, w, txt_len, str(device), frames)
        if key not in self._angles:
            a = longcat_rope_angles(h, w, txt_len, self.cfg.axes_dims_rope, self.cfg.text_position_offset, self.cfg.rope_theta,
                                    frames=frames)
            self._angles[key] = (a.cos().contiguous().to(device), a.sin().contiguous().to(device))
        return self._angles[key]

    def forward(self, hidden_states, encoder_hidden_states, timestep, img_shapes, txt_seq_lens=None, branch: int = 0, **_):
        return super().forward(hidden_states, encoder_hidden_states, timestep, img_shapes, pooled_projections=None,
                               guidance=None, txt_seq_lens=txt_seq_lens, branch=branch)

    def checkpoint_name_map(self) -> dict:
        m = {}
        for k, v in super().checkpoint_name_map().items():
            if k.startswith("time_text_embed.text_embedder") or k.startswith("time_text_embed.guidance_embedder"):
                continue
            m[k.replace("time_text_embed.timestep_embedder.", "time_embed.timestep_embedder.")] = v
        return m
