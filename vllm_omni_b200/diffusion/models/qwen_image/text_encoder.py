"""Qwen2.5-VL language model as the Qwen-Image prompt encoder.

The reference pipeline wraps each prompt in a fixed ChatML template, runs the Hugging Face
``Qwen2_5_VLForConditionalGeneration`` and keeps the last hidden states (after the final norm) of
the tokens that follow the 34-token template head, zero padded per batch with a mask
(vllm_omni/diffusion/models/qwen_image/pipeline_qwen_image.py:292-405).  Here the language model
is this framework's decoder (same kernels as the AR stages): all prompts of a call are packed
into one flat batch of causal prefill segments, so no padding is computed.  For text-only input
the three MRoPE axes carry the same index, i.e. plain rotary positions.

Checkpoint names: ``text_encoder.model.language_model.*`` (or the older ``text_encoder.model.*``);
the vision tower's tensors (``visual.*``) are not needed for text-to-image and are skipped.
"""
from __future__ import annotations

import json
import os

import torch

from ....models.qwen_decoder import DecoderConfig, ModelBatch, PrefillSeg, QwenDecoderModel

PROMPT_TEMPLATE = ("<|im_start|>system\nDescribe the image by detailing the color, shape, size, texture, quantity, text, "
                   "spatial relationships of the objects and background:<|im_end|>\n<|im_start|>user\n{}<|im_end|>\n"
                   "<|im_start|>assistant\n")
TEMPLATE_DROP_TOKENS = 34
TOKENIZER_MAX_LENGTH = 1024


EDIT_TEMPLATE = ("<|im_start|>system\nDescribe the key features of the input image (color, shape, size, texture, objects, "
                 "background), then explain how the user's text instruction should alter or modify the image. Generate a new "
                 "image that meets the user's requirements while maintaining consistency with the original input where "
                 "appropriate.<|im_end|>\n<|im_start|>user\n{}<|im_end|>\n<|im_start|>assistant\n")
EDIT_DROP_TOKENS = 64
IMAGE_SLOT = "<|vision_start|><|image_pad|><|vision_end|>"
CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
CLIP_STD = (0.26862954, 0.26130258, 0.27577711)


def text_config_from_hf(d: dict) -> DecoderConfig:
    """Qwen2.5-VL config.json (flat, or with a ``text_config`` sub-dict) -> decoder geometry.  The
    MRoPE sections are kept: text-only prompts give the three axes the same index (plain rotary
    positions), prompts with images use (t, h, w) triples."""
    t = dict(d.get("text_config") or d)
    t.setdefault("attention_bias", True)          # Qwen2 family: biases on q/k/v, no q/k norm
    t["qk_norm"] = False
    return DecoderConfig.from_dict(t)


def smart_resize(h: int, w: int, factor: int = 28, min_pixels: int = 56 * 56, max_pixels: int = 14 * 14 * 4 * 1280):
    """Target size of the Qwen2-VL image processor: both sides multiples of ``factor``, area inside
    [min_pixels, max_pixels], aspect ratio kept as far as the rounding allows."""
    import math
    hb, wb = max(factor, round(h / factor) * factor), max(factor, round(w / factor) * factor)
    if hb * wb > max_pixels:
        beta = math.sqrt(h * w / max_pixels)
        hb, wb = max(factor, math.floor(h / beta / factor) * factor), max(factor, math.floor(w / beta / factor) * factor)
    elif hb * wb < min_pixels:
        beta = math.sqrt(min_pixels / (h * w))
        hb, wb = math.ceil(h * beta / factor) * factor, math.ceil(w * beta / factor) * factor
    return hb, wb


class QwenVLTextEncoder:
    def __init__(self, cfg: DecoderConfig, tokenizer, dtype=torch.bfloat16, device=None,
                 template: str = PROMPT_TEMPLATE, drop_tokens: int = TEMPLATE_DROP_TOKENS, vision_config=None,
                 image_token_id: int = 151655):
        self.cfg, self.tokenizer = cfg, tokenizer
        self.model = QwenDecoderModel(cfg, dtype, device, with_lm_head=False)
        self.template, self.drop = template, drop_tokens
        self.image_token_id = image_token_id
        self.visual = None
        if vision_config is not None:
            from ....models.qwen2_5_vl_vision import Qwen25VisionTower
            self.visual = Qwen25VisionTower(vision_config, dtype, device)

    @classmethod
    def from_pretrained(cls, model_path: str, dtype=torch.bfloat16, device=None, **kw) -> "QwenVLTextEncoder":
        """``model_path``: a diffusers pipeline directory with ``text_encoder/`` and ``tokenizer/``."""
        from ....engine.tokenizer import get_tokenizer
        with open(os.path.join(model_path, "text_encoder", "config.json")) as f:
            d = json.load(f)
        if kw.pop("with_vision", False) and d.get("vision_config"):
            from ....models.qwen2_5_vl_vision import Qwen25VisionConfig
            kw["vision_config"] = Qwen25VisionConfig.from_dict(d["vision_config"])
            kw["image_token_id"] = int(d.get("image_token_id", 151655))
        return cls(text_config_from_hf(d), get_tokenizer(os.path.join(model_path, "tokenizer")), dtype, device, **kw)

    def to(self, *a, **k):
        self.model.to(*a, **k)
        return self

    @torch.no_grad()
    def __call__(self, prompts: list[str], device=None, dtype=None, max_sequence_length: int | None = None):
        """Returns (states [B, L, D] zero padded, mask [B, L] int64)."""
        dev = self.model.embed_tokens.device
        seqs = []
        for p in prompts:
            ids = self.tokenizer.encode(self.template.format(p), add_special_tokens=False)
            seqs.append(list(ids)[:TOKENIZER_MAX_LENGTH + self.drop])
        flat = torch.tensor([t for s in seqs for t in s], dtype=torch.long, device=dev)
        pos = torch.cat([torch.arange(len(s), device=dev) for s in seqs])
        segs, row = [], 0
        for s in seqs:
            segs.append(PrefillSeg(row, len(s), 0, None))
            row += len(s)
        batch = ModelBatch(flat, pos, torch.full((row,), -1, dtype=torch.int32, device=dev), segs)
        hidden, _ = self.model(batch, None)
        outs, row = [], 0
        for s in seqs:
            outs.append(hidden[row + self.drop:row + len(s)])
            row += len(s)
        L = max(1, max(o.shape[0] for o in outs))
        if max_sequence_length:
            L = min(L, max_sequence_length)
        states = hidden.new_zeros(len(seqs), L, hidden.shape[-1])
        mask = torch.zeros(len(seqs), L, dtype=torch.long, device=dev)
        for i, o in enumerate(outs):
            n = min(L, o.shape[0])
            states[i, :n] = o[:n]
            mask[i, :n] = 1
        return states.to(device=device or dev, dtype=dtype or states.dtype), mask.to(device or dev)

    # ------------------------------------------------------------------ prompts with images (edit pipelines)
    def preprocess_image(self, img: torch.Tensor) -> torch.Tensor:
        """[C, H, W] in [0, 1] -> normalised frames [1, C, H', W'] at the processor's target size."""
        import torch.nn.functional as F
        v = self.visual.cfg
        factor = v.patch_size * v.spatial_merge_size
        H, W = smart_resize(img.shape[-2], img.shape[-1], factor)
        x = F.interpolate(img[None].float(), size=(H, W), mode="bicubic", align_corners=False, antialias=True).clamp(0, 1)
        mean = torch.tensor(CLIP_MEAN, device=x.device).view(1, 3, 1, 1)
        std = torch.tensor(CLIP_STD, device=x.device).view(1, 3, 1, 1)
        return (x - mean) / std

    @torch.no_grad()
    def encode_with_images(self, prompts: list[str], images: list[list[torch.Tensor]], device=None, dtype=None,
                           template: str = EDIT_TEMPLATE, drop_tokens: int = EDIT_DROP_TOKENS, max_sequence_length=None,
                           patches: list[list[tuple]] | None = None):
        """One ``IMAGE_SLOT`` per condition image is put in front of the instruction; every
        ``<|image_pad|>`` token expands to the image's merged patch count, its rows carry the vision
        tower's features and (t, h, w) rotary positions.  ``patches`` may pass pre-cut
        (patch matrix, grid) pairs instead of pixel images.  Returns (states, mask) like ``__call__``."""
        from ....models.mrope import get_input_positions
        if self.visual is None:
            raise RuntimeError("this prompt encoder was built without the vision tower")
        dev = self.model.embed_tokens.device
        emb_table = self.model.embed_tokens
        rows, poss, segs, feats_all, keep = [], [], [], [], []
        row = 0
        for b, prompt in enumerate(prompts):
            pairs = patches[b] if patches is not None else [self.visual.patches_from_pixels(self.preprocess_image(im.to(dev)))
                                                            for im in images[b]]
            feats, grids = [], []
            for pm, grid in pairs:
                f, g = self.visual.forward_patches(pm.to(dev), grid)
                feats.append(f)
                grids.append(g)
            text = template.format(IMAGE_SLOT * len(pairs) + prompt if IMAGE_SLOT not in prompt else prompt)
            ids = list(self.tokenizer.encode(text, add_special_tokens=False))
            out_ids, chunks, k = [], [], 0
            for t in ids:
                if t == self.image_token_id and k < len(feats):
                    out_ids.extend([t] * feats[k].shape[0])
                    chunks.append(feats[k])
                    k += 1
                else:
                    out_ids.append(t)
                    chunks.append(None)
            e = emb_table[torch.tensor(out_ids, device=dev)]
            r = 0
            for t, c in zip([i for i in ids], chunks):
                if c is not None:
                    e[r:r + c.shape[0]] = c.to(e.dtype)
                    r += c.shape[0]
                else:
                    r += 1
            pos, _ = get_input_positions(out_ids, self.image_token_id, -1, -2, list(grids), [])
            rows.append(e)
            poss.append(pos.to(dev))
            segs.append(PrefillSeg(row, len(out_ids), 0, None))
            keep.append(len(out_ids))
            row += len(out_ids)
        x = torch.cat(rows)
        batch = ModelBatch(torch.zeros(row, dtype=torch.long, device=dev), torch.cat(poss, dim=1),
                           torch.full((row,), -1, dtype=torch.int32, device=dev), segs, input_embeds=x)
        hidden, _ = self.model(batch, None)
        outs, r = [], 0
        for n in keep:
            outs.append(hidden[r + drop_tokens:r + n])
            r += n
        L = max(1, max(o.shape[0] for o in outs))
        if max_sequence_length:
            L = min(L, max_sequence_length)
        states = hidden.new_zeros(len(outs), L, hidden.shape[-1])
        mask = torch.zeros(len(outs), L, dtype=torch.long, device=dev)
        for i, o in enumerate(outs):
            n = min(L, o.shape[0])
            states[i, :n], mask[i, :n] = o[:n], 1
        return states.to(device=device or dev, dtype=dtype or states.dtype), mask.to(device or dev)

    @torch.no_grad()
    def load_weights(self, weights) -> set:
        """Names relative to ``text_encoder.``."""
        mapped, back = [], {}
        vis = []
        for n, w in weights:
            if "visual." in n:
                if self.visual is not None:
                    vis.append((n.split("visual.", 1)[1], w, n))
                continue
            if n.startswith("lm_head."):
                continue
            m = n.replace("model.language_model.", "model.", 1) if n.startswith("model.language_model.") else n
            mapped.append((m, w))
            back[m] = n
        loaded = {back[m] for m in self.model.load_weights(mapped)}
        if vis:
            full = {m: n for m, _, n in vis}
            loaded |= {full[m] for m in self.visual.load_weights([(m, w) for m, w, _ in vis])}
        return loaded
