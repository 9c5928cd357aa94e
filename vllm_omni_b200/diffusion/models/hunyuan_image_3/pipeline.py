"""HunyuanImage-3 text-to-image pipeline
(vllm_omni/diffusion/models/hunyuan_image_3/pipeline_hunyuan_image_3.py).

One request builds, per guidance branch, the token sequence
    <bos> prompt <boi> <img_size_B> <img_ratio_i> | <timestep> | <img> x (h*w)
(the unconditional branch replaces every prompt token by <cfg>,
hunyuan_image_3_tokenizer.py:145-151).  Step 0 runs the whole sequence through the MoE decoder
and leaves the prompt's K/V in the per-layer buffers; steps 1.. run only the <timestep> and image
rows against them.  Per step: ``time_embed`` feeds the UNetDown patch embedder that turns the 32
latent channels of every position into a token, ``timestep_emb`` makes the <timestep> token,
``time_embed_2`` feeds the UNetUp head that turns the image rows back into a velocity, and one
fused kernel applies guidance ``u + s (c - u)`` and the flow-match Euler update.  Image sizes snap
to the model's aspect-ratio buckets (hunyuan_image_3_transformer.py:468-553).
"""
from __future__ import annotations

import hashlib
import os

import numpy as np
import torch
from torch import nn

from ....ops import fused
from ...data import DiffusionOutput, OmniDiffusionConfig
from ...schedulers.flow_match_euler import FlowMatchEulerDiscreteScheduler
from ..vae.autoencoder_kl_conv3d import AutoencoderKLConv3D, Conv3dVAEConfig
from .transformer import (HunyuanImage3Config, HunyuanImage3Model, TimestepEmbedder, UNetDown, UNetUp, rope2d_cos_sin,
                          rope2d_positions)


def resolution_buckets(base: int = 1024, step: int | None = None) -> list[tuple[int, int]]:
    """(height, width) buckets sorted by height / width: the square, then height up / width down
    by ``step`` until (2*base, base/2), and the mirror images."""
    step = step or base // 16
    lo, hi = base // 2, base * 2
    out = [(base, base)]
    h, w = base, base
    while not (h >= hi and w <= lo):
        h, w = min(h + step, hi), max(w - step, lo)
        out.append((h, w))
    h, w = base, base
    while not (h <= lo and w >= hi):
        h, w = max(h - step, lo), min(w + step, hi)
        out.append((h, w))
    return sorted(out, key=lambda r: r[0] / r[1])


def snap_resolution(height: int, width: int, base: int = 1024) -> tuple[int, int, int]:
    """(height, width, ratio index) of the bucket whose aspect ratio is nearest."""
    b = resolution_buckets(base)
    i = int(np.argmin([abs(h / w - height / width) for h, w in b]))
    return b[i][0], b[i][1], i


class HunyuanTokens:
    """Special-token ids and prompt encoding.  With the checkpoint's tokenizer the ids are looked
    up by name; without one (random-weight runs) words hash into the lower vocabulary and the
    specials sit at its top."""
    NAMES = ("<boi>", "<eoi>", "<img>", "<cfg>", "<timestep>")

    def __init__(self, vocab_size: int, model_path: str | None = None, base_size: int = 1024):
        self.tok = None
        self.base_size = base_size
        if model_path and os.path.isdir(model_path) and any(
                os.path.isfile(os.path.join(model_path, f)) for f in ("tokenizer.json", "tokenizer_config.json")):
            from transformers import AutoTokenizer
            self.tok = AutoTokenizer.from_pretrained(model_path, trust_remote_code=False)
        if self.tok is not None:
            ids = {n: self.tok.convert_tokens_to_ids(n) for n in self.NAMES}
            self.bos = self.tok.bos_token_id if self.tok.bos_token_id is not None else self.tok.convert_tokens_to_ids("<|startoftext|>")
            self.size_id = self.tok.convert_tokens_to_ids(f"<img_size_{base_size}>")
            self.ratio0 = self.tok.convert_tokens_to_ids("<img_ratio_0>")
        else:
            n_ratio = len(resolution_buckets(base_size))
            top = vocab_size - (len(self.NAMES) + 2 + n_ratio)
            if top < 2:
                raise ValueError(f"vocab_size {vocab_size} leaves no room for the image special tokens")
            ids = {n: top + i for i, n in enumerate(self.NAMES)}
            self.bos, self.size_id, self.ratio0 = top + len(self.NAMES), top + len(self.NAMES) + 1, top + len(self.NAMES) + 2
            self.n_text = top
        self.boi, self.eoi, self.img, self.cfg, self.timestep = (ids[n] for n in self.NAMES)

    def encode(self, text: str, max_len: int) -> list[int]:
        if self.tok is not None:
            return self.tok.encode(text, add_special_tokens=False)[:max_len]
        out = []
        for wd in text.split()[:max_len]:
            out.append(int.from_bytes(hashlib.sha256(wd.encode()).digest()[:4], "little") % self.n_text)
        return out or [0]

    def prompt_rows(self, text: str, ratio_index: int, uncond: bool, max_len: int = 1024) -> list[int]:
        t = self.encode(text, max_len)
        if uncond:
            t = [self.cfg] * len(t)
        return [self.bos] + t + [self.boi, self.size_id, self.ratio0 + ratio_index]


class HunyuanImage3Pipeline(nn.Module):
    default_guidance = 5.0
    flow_shift = 3.0

    def __init__(self, od_config: OmniDiffusionConfig | None = None, transformer_config=None, vae_config=None,
                 device=None, **_):
        super().__init__()
        self.od_config = od_config or OmniDiffusionConfig()
        dtype = self.od_config.dtype
        self.device_ = torch.device(device if device is not None else ("cuda" if torch.cuda.is_available() else "cpu"))
        cfg = transformer_config or HunyuanImage3Config.from_dict(self.od_config.tf_model_config.to_dict())
        self.cfg = cfg
        self.model = HunyuanImage3Model(cfg, dtype, self.device_)
        self.timestep_emb = TimestepEmbedder(cfg.hidden_size, dtype, self.device_)       # the <timestep> token
        self.time_embed = TimestepEmbedder(cfg.hidden_size, dtype, self.device_)         # modulates patch_embed
        self.time_embed_2 = TimestepEmbedder(cfg.hidden_size, dtype, self.device_)       # modulates final_layer
        self.patch_embed = UNetDown(cfg, dtype, self.device_)
        self.final_layer = UNetUp(cfg, dtype, self.device_)
        vc = vae_config if vae_config is not None else (cfg.vae or self.od_config.vae_config)
        vc = Conv3dVAEConfig.from_dict({**(vc or {}), "latent_channels": cfg.latent_channels,
                                        "ffactor_spatial": cfg.vae_downsample}) if not isinstance(vc, Conv3dVAEConfig) else vc
        self.vae = AutoencoderKLConv3D(vc).to(device=self.device_, dtype=dtype)
        self.vae.use_tiling = self.od_config.vae_use_tiling
        self.scheduler = FlowMatchEulerDiscreteScheduler(shift=self.flow_shift, use_dynamic_shifting=False)
        self.tokens = HunyuanTokens(cfg.vocab_size, getattr(self.od_config, "model", None), cfg.image_base_size)
        self.transformer = self.model           # what caches / LoRA / quantisation / TP attach to
        self.vae_decode = None
        self.cfg_exchange = None                # set by CFG-parallel: one guidance branch per rank

    # ------------------------------------------------------------------------------------------
    def _denoise_one(self, text: str, negative: str | None, H: int, W: int, steps: int, scale: float, gen, sigmas=None):
        cfg, dev, dt_ = self.cfg, self.device_, self.od_config.dtype
        f = cfg.vae_downsample * cfg.patch_size
        H, W, ratio = snap_resolution(H, W, cfg.image_base_size) if min(H, W) >= cfg.image_base_size // 2 else (H, W, 0)
        h, w = H // f, W // f
        S = h * w
        do_cfg = scale > 1.0
        branches = [self.tokens.prompt_rows(text, ratio, uncond=False)]
        if do_cfg:
            branches.append(self.tokens.prompt_rows(negative, ratio, uncond=False) if negative
                            else self.tokens.prompt_rows(text, ratio, uncond=True))
        if do_cfg and self.cfg_exchange is not None:
            branches = [branches[1 if self.cfg_exchange.is_negative_rank else 0]]
        nb = len(branches)
        seqs = self.model.begin([len(b) for b in branches], S, dev)
        # rotary tables of the whole sequence, and of the [<timestep>, image] rows the later steps run
        full_cs, tail_cs = [], []
        for b in branches:
            P = len(b)
            c, s = rope2d_cos_sin(rope2d_positions(P + 1 + S, P + 1, h, w), cfg.head_dim, cfg.rope_theta)
            full_cs.append((c, s))
            tail_cs.append((c[P:], s[P:]))
        cat = lambda items, i: torch.cat([it[i] for it in items]).to(dev)
        cs_full, cs_tail = (cat(full_cs, 0), cat(full_cs, 1)), (cat(tail_cs, 0), cat(tail_cs, 1))
        prompt_emb = [self.model.wte[torch.tensor(b, device=dev)] for b in branches]

        z = torch.randn(1, cfg.latent_channels, h, w, generator=gen, device=gen.device if gen is not None else dev)
        lat = z.to(dev, torch.float32).permute(0, 2, 3, 1).reshape(1, S, cfg.latent_channels).contiguous()   # token-major
        lat_in = lat.to(dt_)
        ts = self.scheduler.set_timesteps(steps, device=dev, sigmas=sigmas)
        tv = torch.empty(nb, device=dev)
        for i in range(len(ts)):
            tv.fill_(float(ts[i]))
            x_img = self.patch_embed(lat_in.expand(nb, -1, -1), self.time_embed(tv), h, w)          # [nb, S, D]
            t_tok = self.timestep_emb(tv)                                                           # [nb, D]
            rows = []
            for bi in range(nb):
                if i == 0:
                    rows.append(prompt_emb[bi])
                rows += [t_tok[bi:bi + 1], x_img[bi]]
            hid = self.model(torch.cat(rows).contiguous(), seqs, *(cs_full if i == 0 else cs_tail), first_step=i == 0)
            img_rows, r0 = [], 0
            for s in seqs:
                n = s.total if i == 0 else 1 + s.S
                img_rows.append(hid[r0 + n - S:r0 + n])
                r0 += n
            v = self.final_layer(torch.stack(img_rows), self.time_embed_2(tv), h, w)[..., :cfg.latent_channels]
            dt = self.scheduler.dt(i)
            if do_cfg and self.cfg_exchange is not None:
                self.cfg_exchange.step(v[:1].contiguous(), lat, scale, dt, False, lat_in)
            elif do_cfg:
                fused.cfg_euler_step_(v[:1].contiguous(), v[1:].contiguous(), lat, scale, dt, False, lat_in)
            else:
                fused.cfg_euler_step_(v[:1].contiguous(), None, lat, 1.0, dt, False, lat_in)
        return lat.view(1, h, w, cfg.latent_channels).permute(0, 3, 1, 2), len(ts)

    @torch.no_grad()
    def forward(self, req) -> DiffusionOutput:
        sp = req.sampling_params
        H, W = sp.height or 1024, sp.width or 1024
        gen = sp.generator or (torch.Generator(device="cpu").manual_seed(int(sp.seed)) if sp.seed is not None else None)
        scale = float(sp.guidance_scale if sp.guidance_scale_provided else self.default_guidance)
        lats, n_steps = [], 0
        for p in req.prompts:
            text = p if isinstance(p, str) else p.get("prompt", "")
            neg = None if isinstance(p, str) else p.get("negative_prompt")
            for _ in range(max(1, sp.num_outputs_per_prompt)):
                lat, n_steps = self._denoise_one(text, neg if neg and neg.strip() else None, H, W, sp.num_inference_steps,
                                                 scale, gen, sp.sigmas)
                lats.append(lat)
        lat = torch.cat(lats, 0)
        if (sp.output_type or self.od_config.output_type) == "latent":
            return DiffusionOutput(output=lat)
        img = (self.vae_decode or self.vae.decode)(lat)
        if (img.shape[-2], img.shape[-1]) != (H, W) and min(H, W) < self.cfg.image_base_size // 2:
            img = img[..., :H, :W]
        return DiffusionOutput(output=img, metrics={"num_steps": n_steps, "batch": lat.shape[0]})

    # ------------------------------------------------------------------------------------------
    def load_weights(self, weights) -> set:
        """One flat checkpoint: ``model.*`` (decoder), ``vae.*``, and the five image-side modules by
        their own names; ``lm_head`` and the vision tower of the understanding path are not part of
        text-to-image."""
        heads = {"timestep_emb": self.timestep_emb, "time_embed": self.time_embed, "time_embed_2": self.time_embed_2,
                 "patch_embed": self.patch_embed, "final_layer": self.final_layer}
        params = {k: dict(m.named_parameters()) for k, m in heads.items()}
        dec, vae, loaded = [], [], set()
        for n, w in weights:
            top, _, rest = n.partition(".")
            if top == "model":
                dec.append((n, w))
            elif top == "vae":
                vae.append((rest, w))
            elif top in params:
                p = params[top].get(rest)
                if p is not None and p.shape == w.shape:
                    p.data.copy_(w.to(p.dtype))
                    loaded.add(n)
        loaded |= self.model.load_weights(dec)
        loaded |= {"vae." + n for n in self.vae.load_weights(vae)}
        return loaded
