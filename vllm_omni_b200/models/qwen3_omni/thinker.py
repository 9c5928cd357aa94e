"""Qwen3-Omni thinker stage: MoE decoder with MRoPE, audio and vision towers.

Besides text tokens it emits, per request, the hidden states the talker needs: the input
embeddings ("0"), the output of layer ``accept_hidden_layer`` ("24" in the 30B model) and the
embeddings of the tts bos/eos/pad tokens (vllm_omni/model_executor/models/qwen3_omni/
qwen3_omni_moe_thinker.py:140-186).  They stay on the GPU and travel to the talker stage
through the connector.
"""
from __future__ import annotations

import torch

from ..base import StageModel
from ..mrope import get_input_positions
from ..qwen_decoder import QwenDecoderModel
from .config import Qwen3OmniConfig
from .encoders import AudioEncoder, VisionEncoder


class Qwen3OmniMoeThinker(StageModel):
    engine_output_type = "latent"

    def __init__(self, cfg: Qwen3OmniConfig, dtype=torch.bfloat16, device=None):
        super().__init__(cfg.thinker, dtype, device)
        self.cfg = cfg
        self.decoder = QwenDecoderModel(cfg.thinker, dtype, device)
        self.audio_tower = AudioEncoder(cfg.audio, dtype, device)
        self.visual = VisionEncoder(cfg.vision, dtype, device)
        self.capture = (0, cfg.accept_hidden_layer)

    def eos_token_id(self):
        return self.cfg.im_end_token_id

    def special_token_map(self) -> dict:
        """Marker strings of the chat template and the multimodal placeholders -> token ids of this checkpoint."""
        c = self.cfg
        m = {"<|im_start|>": getattr(c, "im_start_token_id", None), "<|im_end|>": getattr(c, "im_end_token_id", None)}
        for pads, key in ((("<|audio_pad|>", "<|AUDIO|>"), "audio_token_id"), (("<|image_pad|>", "<|IMAGE|>"), "image_token_id"),
                          (("<|video_pad|>", "<|VIDEO|>"), "video_token_id")):     # Qwen3-Omni and Qwen2.5-Omni spellings
            for p in pads:
                m[p] = getattr(c, key, None)
        return {k: v for k, v in m.items() if v is not None}

    @property
    def chunk_stream_keys(self) -> tuple:
        """What a talker that starts before this stage has finished needs from the progress reports: token
        embeddings, the captured hidden layer, and the three TTS marker embeddings (sent once)."""
        return ("0", str(self.cfg.accept_hidden_layer), "tts_bos_embed", "tts_eos_embed", "tts_pad_embed")

    # ---- request preprocessing: multimodal features -> prompt embedding overlay + MRoPE ids
    @torch.no_grad()
    def preprocess_request(self, req) -> None:
        cfg = self.cfg
        mm = req.multi_modal_data or {}
        ids = list(req.prompt_token_ids)
        feats: dict[int, list[torch.Tensor]] = {}
        deep_of: dict[int, list] = {}            # id(feature tensor) -> deep-stack features of that image / video
        image_grids, video_grids = [], []
        dev = self.decoder.embed_tokens.device
        for a in _as_list(mm.get("audio")):
            mel = a[0] if isinstance(a, (tuple, list)) else a            # [n_mels, T] features
            feats.setdefault(cfg.audio_token_id, []).append(self.audio_tower(torch.as_tensor(mel).to(dev)))
        for im in _as_list(mm.get("image")):
            px = torch.as_tensor(im).to(dev)
            px = px[None] if px.dim() == 3 else px
            f, g, deep = self.visual(px)
            feats.setdefault(cfg.image_token_id, []).append(f)
            deep_of[id(f)] = deep
            image_grids.append(g)
        for vd in _as_list(mm.get("video")):
            f, g, deep = self.visual(torch.as_tensor(vd).to(dev))
            feats.setdefault(cfg.video_token_id, []).append(f)
            deep_of[id(f)] = deep
            video_grids.append(g)
        if feats:
            # expand each single placeholder token to the feature length, build the overlay
            new_ids, chunks = [], []
            counters = {k: 0 for k in feats}
            i = 0
            while i < len(ids):
                t = ids[i]
                if t in feats and counters[t] < len(feats[t]):
                    f = feats[t][counters[t]]
                    counters[t] += 1
                    run = 1
                    while i + run < len(ids) and ids[i + run] == t:
                        run += 1
                    new_ids.extend([t] * f.shape[0])
                    chunks.append(("feat", f))
                    i += run
                else:
                    new_ids.append(t)
                    chunks.append(("tok", t))
                    i += 1
            D = cfg.thinker.hidden_size
            emb = torch.empty(len(new_ids), D, dtype=self.dtype_, device=dev)
            r = 0
            tok_rows, tok_ids = [], []
            ds_rows, ds_vals = [], []
            for kind, v in chunks:
                if kind == "feat":
                    emb[r:r + v.shape[0]] = v.to(self.dtype_)
                    if deep_of.get(id(v)):
                        ds_rows.append(torch.arange(r, r + v.shape[0], device=dev))
                        ds_vals.append(deep_of[id(v)])
                    r += v.shape[0]
                else:
                    tok_rows.append(r)
                    tok_ids.append(v)
                    r += 1
            if tok_rows:
                emb[torch.tensor(tok_rows, device=dev)] = self.decoder.embed_tokens[
                    torch.tensor(tok_ids, device=dev).clamp(0, cfg.thinker.vocab_size - 1)]
            req.prompt_token_ids = new_ids
            req.prompt_embeds = emb
            if ds_rows:
                # prompt rows of the visual tokens and, per deep-stack level, their additive features
                levels = len(ds_vals[0])
                req.runtime_state["deepstack"] = (torch.cat(ds_rows), [torch.cat([d[l] for d in ds_vals]).to(self.dtype_)
                                                                       for l in range(levels)])
        pos, _ = get_input_positions(req.prompt_token_ids, cfg.image_token_id, cfg.video_token_id, cfg.audio_token_id,
                                     image_grids, video_grids)
        req.runtime_state["mrope_positions"] = pos

    def positions_for(self, req, start, n):
        mp = req.runtime_state["mrope_positions"]
        L = mp.shape[1]
        if start + n <= L:
            return mp[:, start:start + n]
        nxt = int(mp.max()) + 1
        cols = [mp[:, t] if t < L else torch.full((3,), nxt + (t - L), dtype=torch.long) for t in range(start, start + n)]
        return torch.stack(cols, dim=1)

    def forward_batch(self, batch, kv_caches, sched):
        return self.decoder(batch, kv_caches, capture_layers=self.capture, deepstack=self._deepstack(batch, sched))

    def _deepstack(self, batch, sched):
        """Dense [T, D] additive tensors for this step's rows, one per deep-stack level."""
        out, row = None, 0
        for s in getattr(sched, "scheduled", ()):
            ds = s.request.runtime_state.get("deepstack")
            if ds is not None and s.is_prefill:
                rows, vals = ds
                sel = (rows >= s.start) & (rows < s.start + s.num_new_tokens)
                if bool(sel.any()):
                    if out is None:
                        T, D = batch.input_ids.shape[0], self.cfg.thinker.hidden_size
                        out = [torch.zeros(T, D, dtype=self.dtype_, device=rows.device) for _ in vals]
                    for l, v in enumerate(vals):
                        out[l][rows[sel] - s.start + row] = v[sel]
            row += s.num_new_tokens
        return out

    def collect_outputs(self, sched, batch, hidden, captured) -> None:
        """Append this step's rows of the captured layers to every scheduled request."""
        row = 0
        emb0, hid = captured[0], captured[self.cfg.accept_hidden_layer]
        for s in sched.scheduled:
            r = s.request
            n = s.num_new_tokens
            r.multimodal_outputs.setdefault("0", []).append(emb0[row:row + n])
            r.multimodal_outputs.setdefault(str(self.cfg.accept_hidden_layer), []).append(hid[row:row + n])
            if "tts_bos_embed" not in r.multimodal_outputs:
                c = self.cfg
                e = self.decoder.embed_tokens
                r.multimodal_outputs["tts_bos_embed"] = [e[c.tts_bos_token_id % e.shape[0]][None]]
                r.multimodal_outputs["tts_eos_embed"] = [e[c.tts_eos_token_id % e.shape[0]][None]]
                r.multimodal_outputs["tts_pad_embed"] = [e[c.tts_pad_token_id % e.shape[0]][None]]
            row += n

    @torch.no_grad()
    def load_weights(self, weights):
        """Checkpoint names under ``thinker.``: ``model.*`` / ``lm_head.weight`` (decoder),
        ``audio_tower.*``, ``visual.*``.  Names of other stages are ignored."""
        dec, aud, vis = [], [], []
        for n, w in weights:
            if n.startswith(("talker.", "code2wav.")):
                continue
            m = n[len("thinker."):] if n.startswith("thinker.") else n
            if m.startswith("audio_tower."):
                aud.append((m[len("audio_tower."):], w, n))
            elif m.startswith("visual."):
                vis.append((m[len("visual."):], w, n))
            else:
                dec.append((m, w, n))
        loaded = set()
        for sub, lst in ((self.decoder, dec), (self.audio_tower, aud), (self.visual, vis)):
            full = {m: n for m, _, n in lst}
            loaded |= {full[m] for m in sub.load_weights([(m, w) for m, w, _ in lst])}
        return loaded


def _as_list(x):
    if x is None:
        return []
    return list(x) if isinstance(x, (list, tuple)) and not (len(x) == 2 and isinstance(x[1], (int, float))) else [x]
