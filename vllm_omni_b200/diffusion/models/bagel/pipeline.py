"""BAGEL image generation (vllm_omni/diffusion/models/bagel/pipeline_bagel.py:153-724): the
mixture-of-transformers language model denoises 2x2-patched VAE latents by flow matching while
attending to the key/value cache of the prompt.

Two ways to get that context.  (a) The upstream AR stage prefills the prompt and hands its KV cache
over through the KV transfer manager (``sampling_params.past_key_values``); then, as in the reference,
classifier-free guidance is off.  (b) No cache arrives: this stage tokenizes
``<|im_start|> prompt <|im_end|>`` itself, prefills it in understanding mode, prefills the negative
prompt as the text-CFG context, and samples with text guidance ``v = v_neg + s (v - v_neg)`` inside
the guidance interval, rescaled so that its norm does not exceed the conditional velocity's
(``global`` / ``channel`` / ``text_channel`` renormalisation).

Time grid: ``linspace(1, 0, steps)`` warped by ``shift t / (1 + (shift - 1) t)``, Euler updates
``x -= v dt`` over the first steps - 1 points.  Latent tokens are (h, w) row-major with channel order
(p, q, c); decoding un-patches them and runs the FLUX-layout KL decoder.

Editing (a request with ``multi_modal_data.image``, pipeline_bagel.py:340-520): the reference image is fitted
to the latent stride and enters the context twice in front of the prompt, as clean VAE latents at
timestep 0 (generation weights) and as vision-tower tokens (understanding weights), each block at one
rotary position.  Three contexts feed the guidance: [image, prompt], [image, negative prompt] (text
guidance) and [prompt] alone (image guidance, ``cfg_img_scale`` 1.5 by default); the result has the
fitted size of the reference image.
"""
from __future__ import annotations

import os

import torch
from torch import nn

from ...data import DiffusionOutput, OmniDiffusionConfig
from ..vae import build_vae
from .vision import BagelVisionTower, BagelVitConfig
from .mot import BagelMoT, BagelMoTConfig


def _takes_sample(fn) -> bool:
    import inspect
    try:
        return "sample" in inspect.signature(fn).parameters
    except (TypeError, ValueError):
        return False


def shifted_time_grid(steps: int, shift: float, device=None) -> torch.Tensor:
    t = torch.linspace(1, 0, steps, device=device)
    return shift * t / (1 + (shift - 1) * t)


def guided_velocity(v, v_text=None, v_img=None, text_scale=1.0, img_scale=1.0, renorm_min=0.0, renorm_type="global"):
    """Text (and image) classifier-free guidance with the norm clamp of the reference."""
    if v_text is None or text_scale <= 1.0:
        return v
    if renorm_type == "text_channel":
        vt = v_text + text_scale * (v - v_text)
        scale = (v.norm(dim=-1, keepdim=True) / (vt.norm(dim=-1, keepdim=True) + 1e-8)).clamp(min=renorm_min, max=1.0)
        vt = vt * scale
        return v_img + img_scale * (vt - v_img) if (v_img is not None and img_scale > 1.0) else vt
    vt = v_text + text_scale * (v - v_text)
    out = v_img + img_scale * (vt - v_img) if (v_img is not None and img_scale > 1.0) else vt
    if renorm_type == "global":
        n0, n1 = v.norm(), out.norm()
    elif renorm_type == "channel":
        n0, n1 = v.norm(dim=-1, keepdim=True), out.norm(dim=-1, keepdim=True)
    else:
        raise NotImplementedError(f"{renorm_type} is not supported")
    return out * (n0 / (n1 + 1e-8)).clamp(min=renorm_min, max=1.0)


class BagelPipeline(nn.Module):
    vae_scale_factor = 8

    def __init__(self, od_config: OmniDiffusionConfig | None = None, transformer_config=None, vae_config=None, device=None, **_):
        super().__init__()
        self.od_config = od_config or OmniDiffusionConfig()
        dtype = self.od_config.dtype
        self.device_ = torch.device(device if device is not None else ("cuda" if torch.cuda.is_available() else "cpu"))
        cfg = transformer_config or BagelMoTConfig.from_dict(self.od_config.tf_model_config.to_dict())
        self.transformer = BagelMoT(cfg, dtype=dtype, device=self.device_)
        vc = dict(vae_config or self.od_config.vae_config or {})
        vc.setdefault("latent_channels", cfg.z_channels)
        self.vae = build_vae(vc, "kl", with_encoder=True).to(device=self.device_, dtype=dtype)
        self.vae.use_tiling = self.od_config.vae_use_tiling
        self.tokenizer = None
        self.vae_decode = None
        # vision tower of the editing context (reference image seen by the understanding weights)
        raw = self.od_config.tf_model_config.to_dict() if transformer_config is None else {}
        vit = dict(raw.get("vit_config") or {})
        if "vit_max_num_patch_per_side" in raw:
            vit.setdefault("max_patches_per_side", int(raw["vit_max_num_patch_per_side"]))
        self.vision = BagelVisionTower(BagelVitConfig.from_dict(vit), cfg.hidden_size, dtype=dtype, device=self.device_)

    def attach_text_encoder(self, model_path: str) -> bool:
        """The checkpoint's tokenizer, for prompts that this stage prefills itself."""
        if not any(os.path.exists(os.path.join(model_path, f)) for f in ("tokenizer.json", "tokenizer_config.json", "vocab.json")):
            return False
        from transformers import AutoTokenizer
        self.tokenizer = AutoTokenizer.from_pretrained(model_path)
        c = self.transformer.cfg
        for attr, tok in (("bos_token_id", "<|im_start|>"), ("eos_token_id", "<|im_end|>"), ("start_of_image", "<|vision_start|>"),
                          ("end_of_image", "<|vision_end|>")):
            tid = self.tokenizer.convert_tokens_to_ids(tok)
            if isinstance(tid, int) and tid >= 0 and tid != getattr(self.tokenizer, "unk_token_id", None):
                setattr(c, attr, tid)
        return True

    def load_weights(self, weights) -> set:
        tw, vw = [], []
        for n, w in weights:
            m = n[len("vae."):] if n.startswith("vae.") else (n[len("vae_model."):] if n.startswith("vae_model.") else None)
            if m is not None or n.startswith(("encoder.", "decoder.")):
                vw.append((m if m is not None else n, w))
            else:
                tw.append((n[len("transformer."):] if n.startswith("transformer.") else n, w))
        loaded = set(self.transformer.load_weights(tw)) | set(self.vision.load_weights(tw))
        if vw and hasattr(self.vae, "load_weights"):
            loaded |= {"vae." + n for n in self.vae.load_weights(vw)}
        return loaded

    # ------------------------------------------------------------------ context
    def _prompt_ids(self, text: str) -> torch.Tensor:
        c = self.transformer.cfg
        if self.tokenizer is not None:
            ids = list(self.tokenizer.encode(text, add_special_tokens=False))
        else:                                            # no tokenizer files: bytes of the prompt, a stand-in for tests
            ids = [b % max(1, min(c.vocab_size, 256)) for b in text.encode("utf-8")]
        return torch.tensor([c.bos_token_id] + ids + [c.eos_token_id], dtype=torch.long, device=self.device_)

    def _injected(self, kv):
        """KV handed over by the AR stage -> list of (k, v) [T, Hkv, Dh] per layer."""
        if hasattr(kv, "key_cache"):
            kv = list(zip(kv.key_cache, kv.value_cache))
        L = len(self.transformer.layers)
        out = []
        for li in range(L):
            k, v = kv[li % len(kv)]
            Dh = self.transformer.cfg.head_dim
            out.append((k.to(self.device_).reshape(-1, k.shape[-2], Dh), v.to(self.device_).reshape(-1, v.shape[-2], Dh)))
        return out

    @staticmethod
    def _fit_reference(image, max_side: int, stride: int):
        """Resize rule of the reference for an input image (pipeline_bagel.py:360-383): longest side at most
        ``max_side``, shortest at least 256, both multiples of the latent stride."""
        from PIL import Image
        if isinstance(image, str):
            image = Image.open(image)
        if image.mode != "RGB":
            image = image.convert("RGB")
        w, h = image.size
        scale = min(max_side / max(w, h), 1.0)
        scale = max(scale, min(256, max_side) / min(w, h))
        nw = min(max_side, max(stride, int(round(w * scale / stride) * stride)))
        nh = min(max_side, max(stride, int(round(h * scale / stride) * stride)))
        return image if (nw, nh) == (w, h) else image.resize((nw, nh), Image.BICUBIC)

    def _image_context(self, image, gen=None):
        """Context of an edit: the reference image twice, first as clean VAE latents on the generation
        weights, then as vision-tower tokens on the understanding weights; each takes one rotary position."""
        import numpy as np
        tf, c = self.transformer, self.transformer.cfg
        px = torch.from_numpy(np.asarray(image, dtype=np.float32) / 127.5 - 1.0).permute(2, 0, 1).to(self.device_)
        if _takes_sample(self.vae.encode):               # the reference samples the posterior (bagel/autoencoder.py:274-317)
            g = gen if (gen is not None and gen.device.type == self.device_.type) else None
            z = self.vae.encode(px[None].to(self.od_config.dtype), sample=True, generator=g)
        else:
            z = self.vae.encode(px[None].to(self.od_config.dtype))
        p = c.latent_patch_size
        h, w = z.shape[-2] // p, z.shape[-1] // p
        tok = z[0, :, :h * p, :w * p].reshape(c.z_channels, h, p, w, p).permute(1, 3, 2, 4, 0).reshape(h * w, p * p * c.z_channels)
        ctx = tf.prefill_image_latents(tok.float(), (h, w), None, 0)
        vc = self.vision.cfg
        lim = vc.max_patches_per_side * vc.patch_size
        vw, vh = image.size
        s = min(lim / max(vw, vh), 1.0)
        vw, vh = max(vc.patch_size, int(vw * s) // vc.patch_size * vc.patch_size), max(vc.patch_size, int(vh * s) // vc.patch_size * vc.patch_size)
        from PIL import Image
        vimg = image if (vw, vh) == image.size else image.resize((vw, vh), Image.BICUBIC)
        vpx = torch.from_numpy(np.asarray(vimg, dtype=np.float32) / 127.5 - 1.0).permute(2, 0, 1).to(self.device_)
        ctx = tf.prefill_vision_tokens(self.vision(vpx), ctx, 1)
        return ctx, 2

    # ------------------------------------------------------------------ forward
    @torch.no_grad()
    def forward(self, req) -> DiffusionOutput:
        sp = req.sampling_params
        tf = self.transformer
        c = tf.cfg
        extra = sp.extra_args or {}
        first = req.prompts[0]
        image = (first.get("multi_modal_data") or {}).get("image") if isinstance(first, dict) else None
        if isinstance(image, (list, tuple)):
            image = image[0] if image else None
        if image is not None and sp.past_key_values is not None:
            raise ValueError("a reference image and an injected KV context exclude each other")
        prompt = first if isinstance(first, str) else (first.get("prompt") or "")
        max_hw = c.max_latent_size * c.latent_downsample
        if image is not None:                                # the result has the (stride-aligned) size of the reference image
            image = self._fit_reference(image, max_hw, c.latent_downsample)
            W, H = image.size
        else:
            H = int(sp.height) if sp.height else max_hw
            W = int(sp.width) if sp.width else max_hw
        if H > max_hw or W > max_hw:
            raise ValueError(f"requested {H}x{W} exceeds the checkpoint's limit {max_hw}x{max_hw}")
        h, w = H // c.latent_downsample, W // c.latent_downsample
        steps = int(sp.num_inference_steps or 50)
        text_scale = float(extra.get("cfg_text_scale", 4.0))
        interval = tuple(extra.get("cfg_interval", (0.4, 1.0)))
        renorm_min, renorm_type = float(extra.get("cfg_renorm_min", 0.0)), extra.get("cfg_renorm_type", "global")
        gen = sp.generator or (torch.Generator(device="cpu").manual_seed(int(sp.seed)) if sp.seed is not None else None)
        img_scale = float(extra.get("cfg_img_scale", 1.5 if image is not None else 1.0))
        neg_ctx, neg_pos = None, 0
        img_ctx, img_pos = None, 0                           # image guidance: the prompt WITHOUT the reference image
        if sp.past_key_values is not None:
            ctx = self._injected(sp.past_key_values)
            pos = int(ctx[0][0].shape[0])
            text_scale = 1.0                                 # guidance is off with an injected context
        else:
            ids = self._prompt_ids(prompt)
            neg = first.get("negative_prompt") if isinstance(first, dict) else None
            nids = self._prompt_ids(neg if neg is not None else str(extra.get("negative_prompt", "")))
            base, bpos = (None, 0) if image is None else self._image_context(image, gen)
            ctx, pos = tf.prefill_text(ids, base, bpos), bpos + int(ids.shape[0])
            if text_scale > 1.0:                             # text guidance: same images, the negative prompt
                neg_ctx, neg_pos = tf.prefill_text(nids, base, bpos), bpos + int(nids.shape[0])
            if image is not None and img_scale > 1.0:
                img_ctx, img_pos = tf.prefill_text(ids), int(ids.shape[0])
        x = torch.randn(1, h * w, c.patch_latent_dim, generator=gen, device=gen.device if gen is not None else self.device_)
        x = x.to(self.device_, torch.float32)
        ts = shifted_time_grid(steps, float(extra.get("timestep_shift", c.timestep_shift)), self.device_)
        for i in range(steps - 1):
            t = ts[i]
            v = tf.flow(x, t.reshape(1), (h, w), ctx, pos).float()
            if text_scale > 1.0 and interval[0] < float(t) <= interval[1]:
                vn = tf.flow(x, t.reshape(1), (h, w), neg_ctx, neg_pos, branch=1).float()
                vi = tf.flow(x, t.reshape(1), (h, w), img_ctx, img_pos, branch=2).float() if img_ctx is not None else None
                v = guided_velocity(v, vn, vi, text_scale, img_scale, renorm_min, renorm_type)
            x = x - v * (ts[i] - ts[i + 1])
        p = c.latent_patch_size
        z = torch.einsum("nhwpqc->nchpwq", x.reshape(1, h, w, p, p, c.z_channels)).reshape(1, c.z_channels, h * p, w * p)
        if (sp.output_type or self.od_config.output_type) == "latent":
            return DiffusionOutput(output=z)
        img = (self.vae_decode or self.vae.decode)(z)
        return DiffusionOutput(output=img, metrics={"num_steps": steps - 1})
