"""Qwen-Image text-to-image pipeline on the fused MMDiT.

Control flow of ``QwenImagePipeline.forward`` / ``QwenImageCFGParallelMixin.diffuse``
(vllm_omni/diffusion/models/qwen_image/pipeline_qwen_image.py:539-718,
vllm_omni/diffusion/models/qwen_image/cfg_parallel.py:27-123): encode prompt (or take
``prompt_embeds``), 2x2-pack N(0,1) latents, shifted flow-match sigma schedule, true-CFG
denoising loop with norm rescale, un-pack, VAE decode.

Differences by design: cond and uncond run as ONE batch through the transformer (or on two
ranks under CFG-parallel); guidance mix + norm rescale + Euler update + bf16 re-quantise of
the latents are one kernel; several requests of the same resolution share one loop.
"""
from __future__ import annotations

import hashlib
import time

import numpy as np
import torch
from torch import nn

from ....ops import fused
from ...data import DiffusionOutput, OmniDiffusionConfig
from ...request import OmniDiffusionRequest
from ...schedulers.flow_match_euler import FlowMatchEulerDiscreteScheduler, calculate_shift
from ....utils.safetensors_reader import NvtxRange
from ..vae.autoencoder_kl_qwenimage import AutoencoderKLQwenImage2d, QwenImageVAEConfig
from .transformer import QwenImageTransformer2DModel, QwenImageTransformerConfig

QWEN_IMAGE_SCHEDULER = dict(num_train_timesteps=1000, shift=1.0, use_dynamic_shifting=True, base_shift=0.5,
                            max_shift=0.9, base_image_seq_len=256, max_image_seq_len=8192, shift_terminal=0.02,
                            time_shift_type="exponential")


def pack_latents(lat: torch.Tensor) -> torch.Tensor:
    """[B, C, h, w] -> [B, (h/2)(w/2), 4C] (2x2 patches, channel-major inside a patch)."""
    B, C, h, w = lat.shape
    return lat.view(B, C, h // 2, 2, w // 2, 2).permute(0, 2, 4, 1, 3, 5).reshape(B, (h // 2) * (w // 2), C * 4)


def unpack_latents(lat: torch.Tensor, h: int, w: int) -> torch.Tensor:
    """Inverse of :func:`pack_latents`; h, w are latent (not pixel) sizes."""
    B, _, C4 = lat.shape
    C = C4 // 4
    return lat.view(B, h // 2, w // 2, C, 2, 2).permute(0, 3, 1, 4, 2, 5).reshape(B, C, h, w)


class HashTextEncoder:
    """Stand-in text encoder for random-weight runs: a prompt maps to seeded N(0,1) states.

    Real checkpoints plug a Qwen2.5-VL encoder in through ``pipeline.text_encoder``; the
    diffusion benchmarks feed ``prompt_embeds`` directly and never reach this class.
    """

    def __init__(self, dim: int, max_len: int = 256):
        self.dim, self.max_len = dim, max_len

    def __call__(self, prompts: list[str], device, dtype, max_sequence_length=None):
        L = min(max_sequence_length or self.max_len, self.max_len)
        embs, lens = [], []
        for p in prompts:
            seed = int.from_bytes(hashlib.sha256(p.encode()).digest()[:8], "little") % (2 ** 31)
            g = torch.Generator().manual_seed(seed)
            n = max(1, min(L, len(p.split()) + 4))
            e = torch.zeros(L, self.dim)
            e[:n] = torch.randn(n, self.dim, generator=g)
            embs.append(e)
            lens.append(n)
        mask = torch.zeros(len(prompts), L, dtype=torch.long)
        for i, n in enumerate(lens):
            mask[i, :n] = 1
        return torch.stack(embs).to(device=device, dtype=dtype), mask.to(device)


class QwenImagePipeline(nn.Module):
    vae_scale_factor = 8

    def __init__(self, od_config: OmniDiffusionConfig | None = None, transformer_config=None, vae_config=None,
                 device=None, scheduler_config: dict | None = None):
        super().__init__()
        self.od_config = od_config or OmniDiffusionConfig()
        dtype = self.od_config.dtype
        self.device_ = torch.device(device if device is not None else ("cuda" if torch.cuda.is_available() else "cpu"))
        tcfg = transformer_config or QwenImageTransformerConfig.from_dict(self.od_config.tf_model_config.to_dict())
        self.transformer = QwenImageTransformer2DModel(tcfg, dtype=dtype, device=self.device_)
        self.vae = AutoencoderKLQwenImage2d(vae_config or QwenImageVAEConfig()).to(device=self.device_, dtype=dtype)
        self.vae.use_tiling = self.od_config.vae_use_tiling
        self.scheduler = FlowMatchEulerDiscreteScheduler(**(scheduler_config or QWEN_IMAGE_SCHEDULER))
        self.text_encoder = HashTextEncoder(tcfg.joint_attention_dim)
        self.default_sample_size = 128
        self._loop_cache: dict = {}
        self.cfg_exchange = None        # set by CFG-parallel: fused peer exchange + step
        self.vae_decode = None          # set by VAE patch parallel

    # ------------------------------------------------------------------ helpers
    def encode_prompt(self, prompts, prompt_embeds=None, prompt_embeds_mask=None, max_sequence_length=None):
        if prompt_embeds is not None:
            pe = prompt_embeds.to(self.device_, self.od_config.dtype)
            if pe.dim() == 2:
                pe = pe.unsqueeze(0)
            if prompt_embeds_mask is None:
                prompt_embeds_mask = torch.ones(pe.shape[:2], dtype=torch.long, device=pe.device)
            return pe, prompt_embeds_mask.to(self.device_)
        return self.text_encoder(prompts, self.device_, self.od_config.dtype, max_sequence_length)

    def prepare_latents(self, batch, height, width, generator, latents=None):
        h, w = 2 * (height // (self.vae_scale_factor * 2)), 2 * (width // (self.vae_scale_factor * 2))
        C = self.transformer.cfg.in_channels // 4
        if latents is not None:
            return latents.to(self.device_, torch.float32), h, w
        if isinstance(generator, (list, tuple)):
            z = torch.cat([torch.randn(1, C, h, w, generator=g, device=g.device).to(self.device_) for g in generator])
        else:
            gdev = generator.device if generator is not None else self.device_
            z = torch.randn(batch, C, h, w, generator=generator, device=gdev).to(self.device_)
        return pack_latents(z.float()), h, w

    def prepare_timesteps(self, num_inference_steps, sigmas, image_seq_len):
        sigmas = np.linspace(1.0, 1 / num_inference_steps, num_inference_steps) if sigmas is None else sigmas
        c = self.scheduler.config
        mu = calculate_shift(image_seq_len, c.get("base_image_seq_len", 256), c.get("max_image_seq_len", 4096),
                             c.get("base_shift", 0.5), c.get("max_shift", 1.15))
        return self.scheduler.set_timesteps(sigmas=sigmas, mu=mu, device=self.device_)

    # ------------------------------------------------------------------ denoise
    @torch.no_grad()
    def diffuse(self, prompt_embeds, prompt_mask, neg_embeds, neg_mask, latents, img_shape, timesteps,
                do_true_cfg, true_cfg_scale, cfg_normalize=True, step_callback=None):
        """latents: fp32 [B, S, C] master copy, updated in place and returned."""
        B = latents.shape[0]
        dt_model = self.od_config.dtype
        cfg_par = self.cfg_exchange is not None and do_true_cfg
        if do_true_cfg and not cfg_par:
            # one batch: rows [0,B) conditional, rows [B,2B) unconditional
            L = max(prompt_embeds.shape[1], neg_embeds.shape[1])
            enc = torch.zeros(2 * B, L, prompt_embeds.shape[2], dtype=dt_model, device=latents.device)
            enc[:B, :prompt_embeds.shape[1]] = prompt_embeds
            enc[B:, :neg_embeds.shape[1]] = neg_embeds
            lens = prompt_mask.sum(1).tolist() + neg_mask.sum(1).tolist()
            nb = 2 * B
        elif cfg_par and self.cfg_exchange.is_negative_rank:
            enc, lens, nb = neg_embeds.to(dt_model), neg_mask.sum(1).tolist(), B
        else:
            enc, lens, nb = prompt_embeds.to(dt_model), prompt_mask.sum(1).tolist(), B
        use_graph = not self.od_config.enforce_eager
        full_latents = latents
        sp = self.transformer.sp
        if sp is not None:
            # sequence parallel: this rank keeps S/P image rows and L/P text rows for the whole loop
            P, r = sp.P, sp.rank
            S = latents.shape[1]
            if S % P:
                raise ValueError(f"image tokens ({S}) must be divisible by the sequence-parallel degree ({P})")
            Lp = (enc.shape[1] + P - 1) // P * P
            if Lp != enc.shape[1]:
                enc = torch.nn.functional.pad(enc, (0, 0, 0, Lp - enc.shape[1]))
            enc = enc[:, r * (Lp // P):(r + 1) * (Lp // P)].contiguous()
            latents = latents[:, r * (S // P):(r + 1) * (S // P)].contiguous()
        st = self._loop_state(enc, lens, img_shape, latents.shape[1], len(timesteps), use_graph)
        lat_in = st.lat_in
        lat_in[:B].copy_(latents)
        if nb > B:
            lat_in[B:].copy_(lat_in[:B])
        for i in range(len(timesteps)):
            nvtx = NvtxRange("denoise_step").__enter__()
            v = self.transformer.forward_step(st, i)
            dt = self.scheduler.dt(i)
            if cfg_par:
                self.cfg_exchange.step(v, latents, true_cfg_scale, dt, cfg_normalize, lat_in)
            elif do_true_cfg:
                fused.cfg_euler_step_(v[:B], v[B:], latents, true_cfg_scale, dt, cfg_normalize, lat_in[:B])
                lat_in[B:].copy_(lat_in[:B])
            else:
                fused.cfg_euler_step_(v, None, latents, 1.0, dt, False, lat_in)
            if step_callback is not None:
                step_callback(i, latents)
            nvtx.__exit__(None, None, None)
        if sp is not None:
            parts = sp.group.all_gather(latents, dim=1)       # once per image, before the VAE
            full_latents.copy_(parts)
            latents = full_latents
        return latents

    def _loop_state(self, enc, lens, img_shape, S_img, n_steps, use_graph):
        """Denoising-loop state; the workspace, and with it a captured CUDA graph, is reused
        across requests of the same shape (only the request-dependent tensors are refreshed)."""
        sig = [float(s) for s in self.scheduler.sigmas[:n_steps]]
        key = (tuple(enc.shape), tuple(int(l) for l in lens), tuple(img_shape), S_img, tuple(sig), use_graph)
        fresh = self.transformer.prepare_loop(enc, sig, img_shape, S_img, txt_seq_lens=lens, use_graph=use_graph)
        old = self._loop_cache.get(key)
        if old is None:
            if len(self._loop_cache) >= 4:
                self._loop_cache.pop(next(iter(self._loop_cache)))
            self._loop_cache[key] = fresh
            return fresh
        # same shapes: keep the captured graph and its static buffers, refresh their contents
        old.txt0.copy_(fresh.txt0)
        old.mods_all.copy_(fresh.mods_all)
        old.ss_all.copy_(fresh.ss_all)
        old.temb_all.copy_(fresh.temb_all)
        return old

    # ------------------------------------------------------------------ forward
    @torch.no_grad()
    def forward(self, req: OmniDiffusionRequest) -> DiffusionOutput:
        sp = req.sampling_params
        t0 = time.perf_counter()
        prompts = req.prompts
        texts, negs, pe_list, ne_list = [], [], [], []
        for p in prompts:
            if isinstance(p, str):
                texts.append(p); negs.append(None); pe_list.append(None); ne_list.append(None)
            else:
                texts.append(p.get("prompt", "")); negs.append(p.get("negative_prompt"))
                pe_list.append(p.get("prompt_embeds")); ne_list.append(p.get("negative_prompt_embeds"))
        n_out = sp.num_outputs_per_prompt
        height = sp.height or self.default_sample_size * self.vae_scale_factor
        width = sp.width or self.default_sample_size * self.vae_scale_factor
        true_cfg = sp.true_cfg_scale if sp.true_cfg_scale is not None else (sp.guidance_scale or 1.0)
        has_neg = any(n is not None for n in negs) or any(n is not None for n in ne_list)
        do_true_cfg = true_cfg > 1 and has_neg

        def enc(texts_, embeds_):
            if all(e is not None for e in embeds_):
                es = [e.reshape(-1, e.shape[-1]) for e in embeds_]
                L = max(e.shape[0] for e in es)
                pe = torch.stack([torch.nn.functional.pad(e, (0, 0, 0, L - e.shape[0])) for e in es])
                mask = torch.zeros(len(es), L, dtype=torch.long, device=pe.device)
                for i, e in enumerate(es):
                    mask[i, :e.shape[0]] = 1
                return self.encode_prompt(None, pe, mask)
            return self.encode_prompt([t or "" for t in texts_], max_sequence_length=sp.max_sequence_length)

        pe, pm = enc(texts, pe_list)
        ne = nm = None
        if do_true_cfg:
            ne, nm = enc([n if n is not None else " " for n in negs], ne_list)
        if n_out > 1:
            pe, pm = pe.repeat_interleave(n_out, 0), pm.repeat_interleave(n_out, 0)
            if ne is not None:
                ne, nm = ne.repeat_interleave(n_out, 0), nm.repeat_interleave(n_out, 0)
        B = pe.shape[0]
        gen = sp.generator
        if gen is None and sp.seed is not None:
            gen = torch.Generator(device="cpu").manual_seed(int(sp.seed))
        latents, h, w = self.prepare_latents(B, height, width, gen, sp.latents)
        img_shape = (1, h // 2, w // 2)
        timesteps = self.prepare_timesteps(sp.num_inference_steps, sp.sigmas, latents.shape[1])
        traj = [] if sp.return_trajectory_latents else None
        cb = (lambda i, l: traj.append(l.clone())) if traj is not None else None
        t1 = time.perf_counter()
        latents = self.diffuse(pe, pm, ne, nm, latents, img_shape, timesteps, do_true_cfg, float(true_cfg),
                               cfg_normalize=True, step_callback=cb)
        out_type = sp.output_type if sp.output_type else self.od_config.output_type
        if out_type == "latent":
            image = latents
        else:
            z = unpack_latents(latents, h, w)
            image = (self.vae_decode or self.vae.decode)(z)
        metrics = {"encode_s": t1 - t0, "num_steps": len(timesteps), "batch": B}
        return DiffusionOutput(output=image, trajectory_latents=torch.stack(traj) if traj else None,
                               trajectory_timesteps=list(timesteps) if traj is not None else None, metrics=metrics)

    # ------------------------------------------------------------------ weights
    def load_weights(self, weights) -> set:
        """``weights``: iterable of (name, tensor) with diffusers sub-folder prefixes
        ``transformer.`` / ``vae.``."""
        tw, vw, ew = [], [], []
        for n, w in weights:
            if n.startswith("transformer."):
                tw.append((n[len("transformer."):], w))
            elif n.startswith("vae."):
                vw.append((n[len("vae."):], w))
            elif n.startswith("text_encoder."):
                ew.append((n[len("text_encoder."):], w))
        loaded = {"transformer." + n for n in self.transformer.load_weights(tw)}
        loaded |= {"vae." + n for n in self.vae.load_weights(vw)}
        if ew and hasattr(self.text_encoder, "load_weights"):
            loaded |= {"text_encoder." + n for n in self.text_encoder.load_weights(ew)}
        return loaded

    def attach_text_encoder(self, model_path: str) -> bool:
        """Replace the stand-in prompt encoder by the checkpoint's Qwen2.5-VL language model when the
        pipeline directory carries ``text_encoder/`` and ``tokenizer/``."""
        import os
        if not (os.path.isfile(os.path.join(model_path, "text_encoder", "config.json")) and
                os.path.isdir(os.path.join(model_path, "tokenizer"))):
            return False
        from .text_encoder import QwenVLTextEncoder
        self.text_encoder = QwenVLTextEncoder.from_pretrained(model_path, self.od_config.dtype, self.device_)
        return True
