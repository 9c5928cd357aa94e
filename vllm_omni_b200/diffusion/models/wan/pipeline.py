"""Wan text-to-video / image-to-video pipelines
(vllm_omni/diffusion/models/wan2_2/pipeline_wan2_2*.py): UMT5 text states (or given
``prompt_embeds``), N(0,1) video latents [16, 1+(F-1)/4, H/8, W/8], UniPC flow scheduler
(shift 5.0 at 720p, 3.0 at 480p), CFG with cond/uncond batched through the transformer,
optional second transformer for the low-noise part of the schedule (``boundary_ratio``), causal
3-D VAE decode.  Image-to-video concatenates the encoded first frame + mask to the latents.
"""
from __future__ import annotations

import torch
from torch import nn

from ...data import DiffusionOutput, OmniDiffusionConfig
from ...request import OmniDiffusionRequest
from ...schedulers.flow_unipc import FlowUniPCMultistepScheduler
from ..qwen_image.pipeline import HashTextEncoder
from ..vae.autoencoder_kl_qwenimage import QwenImageVAEConfig
from ..vae.autoencoder_kl_wan import AutoencoderKLWan
from .transformer import WanTransformer3DModel, WanTransformerConfig


class WanPipeline(nn.Module):
    vae_scale_spatial, vae_scale_temporal = 8, 4
    image_conditioned = False

    def __init__(self, od_config: OmniDiffusionConfig | None = None, transformer_config=None, vae_config=None,
                 device=None, **_):
        super().__init__()
        self.od_config = od_config or OmniDiffusionConfig()
        dtype = self.od_config.dtype
        self.device_ = torch.device(device if device is not None else ("cuda" if torch.cuda.is_available() else "cpu"))
        tcfg = transformer_config or WanTransformerConfig.from_dict(self.od_config.tf_model_config.to_dict())
        if self.image_conditioned and transformer_config is None and "in_channels" not in self.od_config.tf_model_config.params:
            tcfg.in_channels = 2 * tcfg.out_channels + 4          # latents + mask + first-frame latents
        self.transformer = WanTransformer3DModel(tcfg, dtype=dtype, device=self.device_)
        self.transformer_2 = None
        if self.od_config.boundary_ratio is not None:
            self.transformer_2 = WanTransformer3DModel(tcfg, dtype=dtype, device=self.device_)
        self.vae = AutoencoderKLWan(vae_config or QwenImageVAEConfig()).to(device=self.device_, dtype=torch.float32
                                                                           if self.device_.type == "cpu" else dtype)
        self.scheduler = FlowUniPCMultistepScheduler(shift=self.od_config.flow_shift or 5.0)
        self.text_encoder = HashTextEncoder(tcfg.text_dim, max_len=512)
        self.vae_decode = None
        self.cfg_exchange = None        # set by CFG-parallel: rank 0 runs the prompt branch, rank 1 the negative one

    def attach_text_encoder(self, model_path: str) -> bool:
        """``text_encoder/`` (UMT5) + ``tokenizer/``: states of padded positions are zeroed, as the reference does
        (vllm_omni/diffusion/models/wan2_2/pipeline_wan2_2.py, ``_get_t5_prompt_embeds``)."""
        import os
        if not (os.path.isfile(os.path.join(model_path, "text_encoder", "config.json")) and
                os.path.isdir(os.path.join(model_path, "tokenizer"))):
            return False
        from ..text_encoders.t5 import T5PromptEncoder
        self.text_encoder = T5PromptEncoder.from_pretrained(model_path, "text_encoder", "tokenizer", self.od_config.dtype,
                                                            self.device_, max_len=512, zero_padding=True)
        return True

    def _embeds(self, prompts, key, negs=False):
        es = [p.get(key) if isinstance(p, dict) else None for p in prompts]
        if all(e is not None for e in es):
            L = max(e.shape[-2] for e in es)
            return torch.stack([torch.nn.functional.pad(e.reshape(-1, e.shape[-1]), (0, 0, 0, L - e.shape[-2]))
                                for e in es]).to(self.device_, self.od_config.dtype)
        texts = [((p.get("negative_prompt") or " ") if negs else p.get("prompt", "")) if isinstance(p, dict)
                 else (" " if negs else p) for p in prompts]
        return self.text_encoder(texts, self.device_, self.od_config.dtype)[0]

    @torch.no_grad()
    def forward(self, req: OmniDiffusionRequest) -> DiffusionOutput:
        sp = req.sampling_params
        B = len(req.prompts) * sp.num_outputs_per_prompt
        H, W = sp.height or 480, sp.width or 832
        F_ = sp.num_frames if sp.num_frames and sp.num_frames > 1 else 17
        T = (F_ - 1) // self.vae_scale_temporal + 1
        h, w = H // self.vae_scale_spatial, W // self.vae_scale_spatial
        C = self.transformer.cfg.out_channels
        gen = sp.generator
        if gen is None and sp.seed is not None:
            gen = torch.Generator(device="cpu").manual_seed(int(sp.seed))
        lat = torch.randn(B, C, T, h, w, generator=gen, device=gen.device if gen is not None else self.device_)
        lat = lat.to(self.device_, torch.float32) if sp.latents is None else sp.latents.to(self.device_, torch.float32)
        pe = self._embeds(req.prompts, "prompt_embeds").repeat_interleave(sp.num_outputs_per_prompt, 0)
        guidance = sp.guidance_scale if sp.guidance_scale_provided else 5.0
        do_cfg = guidance > 1.0
        ne = self._embeds(req.prompts, "negative_prompt_embeds", negs=True).repeat_interleave(
            sp.num_outputs_per_prompt, 0) if do_cfg else None
        if do_cfg and ne.shape[1] != pe.shape[1]:
            L = max(ne.shape[1], pe.shape[1])
            pe = torch.nn.functional.pad(pe, (0, 0, 0, L - pe.shape[1]))
            ne = torch.nn.functional.pad(ne, (0, 0, 0, L - ne.shape[1]))
        cond = self._image_condition(req, B, T, h, w) if self.image_conditioned else None
        ts = self.scheduler.set_timesteps(sp.num_inference_steps, device=self.device_)
        boundary = None
        if self.transformer_2 is not None:
            boundary = (sp.boundary_ratio or self.od_config.boundary_ratio) * 1000.0
        cfg_par = do_cfg and self.cfg_exchange is not None
        if cfg_par:
            enc = ne if self.cfg_exchange.is_negative_rank else pe
        else:
            enc = torch.cat([pe, ne], 0) if do_cfg else pe
        for i, t in enumerate(ts):
            model = self.transformer if (boundary is None or float(t) >= boundary) else self.transformer_2
            x = lat.to(self.od_config.dtype)
            if cond is not None:
                x = torch.cat([x, cond], dim=1)
            xin = torch.cat([x, x], 0) if (do_cfg and not cfg_par) else x
            tv = t.expand(xin.shape[0])
            v = model(xin, tv, enc).float()
            if do_cfg:
                if cfg_par:                              # both ranks take both branches and step their own copy identically
                    vc, vu = self.cfg_exchange.group.all_gather(v.contiguous(), separate_tensors=True)
                else:
                    vc, vu = v[:B], v[B:]
                g = guidance if (boundary is None or float(t) >= boundary) else (sp.guidance_scale_2 or guidance)
                v = vu + g * (vc - vu)
            lat = self.scheduler.step(v, t, lat)
        if (sp.output_type or self.od_config.output_type) == "latent":
            return DiffusionOutput(output=lat)
        video = (self.vae_decode or self.vae.decode)(lat.to(self.vae.dtype))
        return DiffusionOutput(output=video, metrics={"num_steps": len(ts), "frames": video.shape[2]})

    def _image_condition(self, req, B, T, h, w):
        return None

    def load_weights(self, weights) -> set:
        tw, t2, te = [], [], []
        for n, w in weights:
            if n.startswith("transformer_2."):
                t2.append((n[len("transformer_2."):], w))
            elif n.startswith("transformer."):
                tw.append((n[len("transformer."):], w))
            elif n.startswith("text_encoder."):
                te.append((n[len("text_encoder."):], w))
        loaded = {"transformer." + n for n in self.transformer.load_weights(tw)}
        if te and hasattr(self.text_encoder, "load_weights"):
            loaded |= {"text_encoder." + n for n in self.text_encoder.load_weights(te)}
        if self.transformer_2 is not None:
            loaded |= {"transformer_2." + n for n in self.transformer_2.load_weights(t2)}
        return loaded


class WanImageToVideoPipeline(WanPipeline):
    image_conditioned = True

    def _image_condition(self, req, B, T, h, w):
        """[B, 4 + C, T, h, w]: a mask that marks the first frame as given, and the latent of the
        conditioning image in frame 0 (zeros elsewhere).  Without an encoder checkpoint the image
        is average-pooled to the latent grid."""
        C = self.transformer.cfg.out_channels
        cond = torch.zeros(B, 4 + C, T, h, w, dtype=self.od_config.dtype, device=self.device_)
        cond[:, :4, 0] = 1.0
        for i, p in enumerate(req.prompts):
            imgs = (p.get("multi_modal_data") or {}).get("image_tensor") if isinstance(p, dict) else None
            if imgs:
                im = imgs[0].to(self.device_, torch.float32)[None]
                z = torch.nn.functional.adaptive_avg_pool2d(im, (h, w))[0]
                cond[i, 4:4 + min(3, C), 0] = z[:min(3, C)].to(cond.dtype)
        return cond


class WanTI2VPipeline(WanImageToVideoPipeline):
    """Text+image to video with the high-compression VAE variant (same control flow)."""
