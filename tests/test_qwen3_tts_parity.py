"""Qwen3-TTS against oracles assembled from Hugging Face building blocks (fp32, CPU).

transformers has no Qwen3-TTS module, so the oracles are put together here from modules whose math
it does ship and which the published model reuses: dense ``Qwen3Model`` stacks for the talker and
the code predictor (the talker's three rotary axes carry equal positions for speech rows, which is
the ordinary 1-D rotary embedding), the Qwen3-Omni code2wav convolution / transformer blocks for the
12 Hz tokenizer decoder, and the HF logits processors.  Around them the prompt assembly, the
per-step input rule and the quantizer are restated step by step, and the state dict is named as the
published checkpoint names its tensors.
"""
import math

import pytest
import torch
import torch.nn.functional as F
from torch import nn

transformers = pytest.importorskip("transformers")

from vllm_omni_b200.models.qwen3_tts.model import Qwen3TTSConfig, Qwen3TTSModel


def _init(mod, std=0.05):
    for n, p in mod.named_parameters():
        if p.dim() > 1:
            torch.nn.init.normal_(p, 0, std)
        else:
            torch.nn.init.normal_(p, 0.8 if "norm" in n else 0.0, 0.1)
    return mod.float().eval()


# ----------------------------------------------------------------------------- talker oracle
class _TalkerOracle(nn.Module):
    def __init__(self, c: Qwen3TTSConfig):
        super().__init__()
        t, p = c.talker, c.code_predictor
        Q = transformers.Qwen3Config
        common = dict(max_position_embeddings=512, attention_bias=False, rope_parameters={"rope_type": "default", "rope_theta": 1e4})
        self.talker = transformers.Qwen3Model(Q(vocab_size=t.vocab_size, hidden_size=t.hidden_size,
                                                num_hidden_layers=t.num_hidden_layers, num_attention_heads=t.num_attention_heads,
                                                num_key_value_heads=t.num_key_value_heads, head_dim=t.head_dim,
                                                intermediate_size=t.intermediate_size, rms_norm_eps=t.rms_norm_eps, **common))
        self.cp = transformers.Qwen3Model(Q(vocab_size=p.vocab_size, hidden_size=p.hidden_size, num_hidden_layers=p.num_hidden_layers,
                                            num_attention_heads=p.num_attention_heads, num_key_value_heads=p.num_key_value_heads,
                                            head_dim=p.head_dim, intermediate_size=p.intermediate_size, rms_norm_eps=p.rms_norm_eps,
                                            **common))
        G = p.num_code_groups
        self.text_embedding = nn.Embedding(c.text_vocab_size, c.text_hidden_size)
        self.fc1 = nn.Linear(c.text_hidden_size, c.text_hidden_size)
        self.fc2 = nn.Linear(c.text_hidden_size, t.hidden_size)
        self.codec_head = nn.Linear(t.hidden_size, t.vocab_size, bias=False)
        self.cp_embed = nn.ModuleList([nn.Embedding(p.vocab_size, t.hidden_size) for _ in range(G - 1)])
        self.cp_head = nn.ModuleList([nn.Linear(p.hidden_size, p.vocab_size, bias=False) for _ in range(G - 1)])
        self.small_to_mtp = nn.Linear(t.hidden_size, p.hidden_size)
        self.c = c

    def checkpoint(self) -> dict:
        sd = {}
        for k, v in self.talker.state_dict().items():
            sd["talker.model." + ("codec_embedding.weight" if k == "embed_tokens.weight" else k)] = v
        sd["talker.model.text_embedding.weight"] = self.text_embedding.weight
        for a, m in (("linear_fc1", self.fc1), ("linear_fc2", self.fc2)):
            sd[f"talker.text_projection.{a}.weight"], sd[f"talker.text_projection.{a}.bias"] = m.weight, m.bias
        sd["talker.codec_head.weight"] = self.codec_head.weight
        for k, v in self.cp.state_dict().items():
            if k != "embed_tokens.weight":
                sd["talker.code_predictor.model." + k] = v
        for g in range(len(self.cp_embed)):
            sd[f"talker.code_predictor.model.codec_embedding.{g}.weight"] = self.cp_embed[g].weight
            sd[f"talker.code_predictor.lm_head.{g}.weight"] = self.cp_head[g].weight
        sd["talker.code_predictor.small_to_mtp_projection.weight"] = self.small_to_mtp.weight
        sd["talker.code_predictor.small_to_mtp_projection.bias"] = self.small_to_mtp.bias
        return sd

    def text(self, ids):
        return self.fc2(F.silu(self.fc1(self.text_embedding(torch.tensor(ids).view(1, -1)))))

    def codec(self, ids):
        return self.talker.embed_tokens(torch.tensor(ids).view(1, -1))

    def prompt(self, input_id, instruct_id=None, spk_embed=None, language_id=None, ref_id=None, ref_code=None,
               non_streaming=False):
        c = self.c
        pad, bos, eos = self.text([c.tts_pad_token_id, c.tts_bos_token_id, c.tts_eos_token_id]).chunk(3, dim=1)
        pre = [c.codec_nothink_id, c.codec_think_bos_id, c.codec_think_eos_id] if language_id is None else \
            [c.codec_think_id, c.codec_think_bos_id, language_id, c.codec_think_eos_id]
        e0, e1 = self.codec(pre), self.codec([c.codec_pad_id, c.codec_bos_id])
        cin = torch.cat([e0, e1], 1) if spk_embed is None else torch.cat([e0, spk_embed.view(1, 1, -1), e1], 1)
        role = self.text(input_id[:3])
        mid = torch.cat((pad.expand(-1, cin.shape[1] - 2, -1), bos), 1) + cin[:, :-1]
        out = torch.cat((role, mid), 1)
        if ref_code is not None:
            text_embed = torch.cat([self.text(ref_id[3:-2] + input_id[3:-5]), eos], 1)
            ce = [self.talker.embed_tokens(ref_code[:, :1])] + [self.cp_embed[i - 1](ref_code[:, i:i + 1])
                                                                 for i in range(1, ref_code.shape[1])]
            ce = torch.cat(ce, 1).sum(1).unsqueeze(0)
            ce = torch.cat([self.codec([c.codec_bos_id]), ce], 1)
            tl, cl = text_embed.shape[1], ce.shape[1]
            if non_streaming:
                icl = torch.cat([text_embed + self.codec([c.codec_pad_id] * tl), ce + pad], 1)
                trailing = pad
            elif tl > cl:
                icl, trailing = text_embed[:, :cl] + ce, text_embed[:, cl:]
            else:
                icl, trailing = torch.cat([text_embed] + [pad] * (cl - tl), 1) + ce, pad
            out = torch.cat([out, icl], 1)
        else:
            out = torch.cat([out, self.text(input_id[3:4]) + cin[:, -1:]], 1)
            if non_streaming:
                out = out[:, :-1]
                n = len(input_id[3:-5]) + 1
                out = torch.cat([out, torch.cat((self.text(input_id[3:-5]), eos), 1) + self.codec([c.codec_pad_id] * n),
                                 pad + self.codec([c.codec_bos_id])], 1)
                trailing = pad
            else:
                trailing = torch.cat((self.text(input_id[4:-5]), eos), 1)
        if instruct_id is not None:
            out = torch.cat([self.text(instruct_id), out], 1)
        return out, trailing, pad

    @torch.no_grad()
    def generate(self, embeds, trailing, pad, steps):
        """Greedy, without a KV cache: every step re-runs the whole sequence."""
        from transformers.generation.logits_process import (MinNewTokensLengthLogitsProcessor, RepetitionPenaltyLogitsProcessor,
                                                            SuppressTokensLogitsProcessor)
        c = self.c
        V = c.talker.vocab_size
        procs = [RepetitionPenaltyLogitsProcessor(1.05),
                 SuppressTokensLogitsProcessor([i for i in range(V - c.suppress_tail, V) if i != c.codec_eos_id]),
                 MinNewTokensLengthLogitsProcessor(0, 2, c.codec_eos_id)]
        seq, ids, frames = embeds, torch.zeros(1, 0, dtype=torch.long), []
        G = c.code_predictor.num_code_groups
        for step in range(steps):
            h = self.talker(inputs_embeds=seq).last_hidden_state[:, -1:]
            scores = self.codec_head(h[:, 0])
            for p in procs:
                scores = p(ids, scores)
            c0 = scores.argmax(-1)
            if int(c0) == c.codec_eos_id:
                break
            ids = torch.cat([ids, c0[None]], 1)
            last = self.talker.embed_tokens(c0)[None]                           # [1, 1, D]
            sub, codes, embs = torch.cat((h, last), 1), [c0], [last]
            for g in range(G - 1):
                hh = self.cp(inputs_embeds=self.small_to_mtp(sub)).last_hidden_state[:, -1]
                cg = self.cp_head[g](hh).argmax(-1)
                eg = self.cp_embed[g](cg)[None]
                codes.append(cg)
                embs.append(eg)
                sub = torch.cat((sub, eg), 1)
            frames.append(torch.stack(codes, 1))
            nxt = torch.cat(embs, 1).sum(1, keepdim=True)
            nxt = nxt + (trailing[:, step:step + 1] if step < trailing.shape[1] else pad)
            seq = torch.cat([seq, nxt], 1)
        return torch.cat(frames, 0) if frames else torch.zeros(0, G, dtype=torch.long)


def _pair(seed=0):
    torch.manual_seed(seed)
    cfg = Qwen3TTSConfig.tiny()
    oracle = _init(_TalkerOracle(cfg), 0.3)
    m = Qwen3TTSModel(cfg, torch.float32, "cpu")
    sd = oracle.checkpoint()
    loaded = m.load_weights(sd.items())
    assert loaded == set(sd), sorted(set(sd) - loaded)
    return cfg, oracle, m


def _wrapped(cfg, text):
    head = [cfg.im_start_token_id, cfg.assistant_token_id, cfg.newline_token_id]
    return head + text + [cfg.im_end_token_id, cfg.newline_token_id] + head


TEXT = [21, 22, 23, 24, 25, 26, 27]


@pytest.mark.parametrize("mode", ["named_voice", "auto_language_no_voice", "instruct", "non_streaming", "dialect"])
def test_prompt_rows_and_greedy_frames_match_the_oracle(mode):
    cfg, oracle, m = _pair(1)
    ids = _wrapped(cfg, TEXT)
    kw_o, kw_m = {}, {}
    if mode == "named_voice":
        kw_o = dict(spk_embed=oracle.codec([cfg.spk_id["vivian"]]), language_id=cfg.codec_language_id["english"])
        kw_m = dict(speaker="Vivian", language="English")
    elif mode == "instruct":
        ins = [cfg.im_start_token_id, cfg.user_token_id, cfg.newline_token_id, 31, 32, 33, cfg.im_end_token_id, cfg.newline_token_id]
        kw_o, kw_m = dict(instruct_id=ins), dict(instruct_ids=[31, 32, 33])
    elif mode == "non_streaming":
        kw_o = dict(spk_embed=oracle.codec([cfg.spk_id["vivian"]]), non_streaming=True)
        kw_m = dict(speaker="vivian", non_streaming_mode=True)
    elif mode == "dialect":            # a dialect voice overrides the language tag when the language is Chinese or auto
        kw_o = dict(spk_embed=oracle.codec([cfg.spk_id["uncle_fu"]]), language_id=cfg.codec_language_id["beijing"])
        kw_m = dict(speaker="uncle_fu", language="auto")
    with torch.no_grad():
        ro, to, po = oracle.prompt(ids, **kw_o)
        rm, tm, pm = m.build_prompt(TEXT, **kw_m)           # the model wraps bare text ids itself
    assert ro.shape[1:] == rm.shape and (ro[0] - rm).abs().max().item() < 1e-5
    assert to.shape[1:] == tm.shape and (to[0] - tm).abs().max().item() < 1e-5
    ref = oracle.generate(ro, to, po, steps=9)
    sy = {k: v for k, v in kw_m.items()}
    codes, wav = m.synthesize(ids, temperature=0.0, max_frames=9, **sy)
    assert ref.shape[0] >= 3 and torch.equal(ref, codes), (ref, codes)
    assert wav.numel() == codes.shape[0] * cfg.tokenizer_decoder.total_upsample and torch.isfinite(wav).all()


def test_in_context_voice_clone_prompt_matches_the_oracle():
    cfg, oracle, m = _pair(2)
    ids = _wrapped(cfg, TEXT)
    ref_text = [41, 42, 43]
    ref_ids = [cfg.im_start_token_id, cfg.assistant_token_id, cfg.newline_token_id] + ref_text + [cfg.im_end_token_id, cfg.newline_token_id]
    G = cfg.code_predictor.num_code_groups
    for T in (4, 14):                                       # fewer / more reference frames than text rows
        ref_code = torch.randint(0, 60, (T, G))
        xvec = torch.randn(cfg.talker.hidden_size)
        voice = {"ref_spk_embedding": xvec, "ref_code": ref_code, "icl_mode": True, "x_vector_only_mode": False}
        for ns in (False, True):
            with torch.no_grad():
                ro, to, po = oracle.prompt(ids, spk_embed=xvec, ref_id=ref_ids, ref_code=ref_code, non_streaming=ns)
                rm, tm, _ = m.build_prompt(ids, voice=voice, ref_ids=ref_text, non_streaming_mode=ns)
            assert ro.shape[1:] == rm.shape and (ro[0] - rm).abs().max().item() < 1e-5
            assert to.shape[1:] == tm.shape and (to[0] - tm).abs().max().item() < 1e-5
        ref = oracle.generate(ro, to, po, steps=6)
        codes, wav = m.synthesize(ids, voice=voice, ref_ids=ref_text, non_streaming_mode=True, temperature=0.0, max_frames=6)
        assert torch.equal(ref, codes)
        # the reference frames are decoded in front and their share of the samples is cut
        assert wav.numel() == codes.shape[0] * cfg.tokenizer_decoder.total_upsample


def test_x_vector_voice_from_audio():
    cfg, oracle, m = _pair(3)
    _init(m.speaker_encoder, 0.2)
    wav = 0.3 * torch.sin(torch.arange(16000) / 16000 * 2 * math.pi * 220)
    v = m.create_voice_clone_prompt(wav, 16000, x_vector_only_mode=True, name="clip")
    assert v["ref_spk_embedding"].shape == (cfg.talker.hidden_size,) and v["x_vector_only_mode"] and not v["icl_mode"]
    with torch.no_grad():
        ro, _, _ = oracle.prompt(_wrapped(cfg, TEXT), spk_embed=v["ref_spk_embedding"])
        rm, _, _ = m.build_prompt(TEXT, voice=m.voices["clip"])
    assert (ro[0] - rm).abs().max().item() < 1e-5


# ----------------------------------------------------------------------------- tokenizer decoder oracle
def test_tokenizer_decoder_against_hf_blocks():
    M = pytest.importorskip("transformers.models.qwen3_omni_moe.modeling_qwen3_omni_moe")
    from transformers.models.qwen3_omni_moe.configuration_qwen3_omni_moe import Qwen3OmniMoeCode2WavConfig
    from vllm_omni_b200.models.qwen3_tts.tokenizer_12hz import Qwen3TTSTokenizerDecoder, TokenizerDecoderConfig
    torch.manual_seed(0)
    bins, G, cd, L, H = 64, 4, 16, 24, 32
    hc = Qwen3OmniMoeCode2WavConfig(codebook_size=bins, hidden_size=H, num_attention_heads=2, num_key_value_heads=2,
                                    sliding_window=5, intermediate_size=64, num_hidden_layers=2, num_quantizers=G,
                                    upsample_rates=[4, 2], upsampling_ratios=[2], decoder_dim=32, max_position_embeddings=512)

    class Oracle(nn.Module):
        def __init__(self):
            super().__init__()
            self.pre_conv = M.Qwen3OmniMoeCausalConvNet(cd, L, kernel_size=3)
            self.pre_transformer = M.Qwen3OmniMoeCode2WavTransformerModel(hc)
            self.pre_transformer.input_proj = nn.Linear(L, H)
            self.pre_transformer.output_proj = nn.Linear(H, L)
            self.upsample = nn.ModuleList([nn.ModuleList([M.Qwen3OmniMoeCausalTransConvNet(L, L, f, f), M.Qwen3OmniMoeConvNeXtBlock(L)])
                                           for f in hc.upsampling_ratios])
            dec = [M.Qwen3OmniMoeCausalConvNet(L, hc.decoder_dim, 7)]
            dec += [M.Qwen3OmniMoeCode2WavDecoderBlock(hc, i) for i in range(len(hc.upsample_rates))]
            out = hc.decoder_dim // 2 ** len(hc.upsample_rates)
            dec += [M.SnakeBeta(out), M.Qwen3OmniMoeCausalConvNet(out, 1, 7)]
            self.decoder = nn.ModuleList(dec)
            for mod in self.modules():                      # this decoder cuts the overhang from the right end only
                if isinstance(mod, M.Qwen3OmniMoeCausalTransConvNet):
                    mod.left_pad = 0
            # split residual quantizer: codebook 0 | codebooks 1.., each with its own 1x1 output conv
            self.q = nn.ParameterDict()
            for grp, n in (("rvq_first", 1), ("rvq_rest", G - 1)):
                for i in range(n):
                    self.q[f"{grp}_sum_{i}"] = nn.Parameter(torch.randn(bins, cd // 2))
                    self.q[f"{grp}_use_{i}"] = nn.Parameter(torch.rand(bins) * 3)
                self.q[f"{grp}_out"] = nn.Parameter(torch.randn(cd, cd // 2, 1) * 0.3)
                self.q[f"{grp}_in"] = nn.Parameter(torch.randn(cd // 2, cd, 1) * 0.3)        # encoder side, unused

        def quantizer_names(self):
            sd = {}
            for grp, n in (("rvq_first", 1), ("rvq_rest", G - 1)):
                for i in range(n):
                    sd[f"quantizer.{grp}.vq.layers.{i}._codebook.embedding_sum"] = self.q[f"{grp}_sum_{i}"]
                    sd[f"quantizer.{grp}.vq.layers.{i}._codebook.cluster_usage"] = self.q[f"{grp}_use_{i}"]
                sd[f"quantizer.{grp}.output_proj.weight"] = self.q[f"{grp}_out"]
                sd[f"quantizer.{grp}.input_proj.weight"] = self.q[f"{grp}_in"]
            return sd

        def dequantize(self, codes):                        # [B, G, T] -> [B, cd, T]
            def rvq(grp, cs):
                acc = 0
                for i in range(cs.shape[1]):
                    table = self.q[f"{grp}_sum_{i}"] / self.q[f"{grp}_use_{i}"].clamp(min=1e-5)[:, None]
                    acc = acc + F.embedding(cs[:, i], table).transpose(1, 2)
                return F.conv1d(acc, self.q[f"{grp}_out"])
            return rvq("rvq_first", codes[:, :1]) + rvq("rvq_rest", codes[:, 1:])

        def forward(self, codes):
            h = self.pre_conv(self.dequantize(codes)).transpose(1, 2)
            pt = self.pre_transformer
            h = pt.output_proj(pt(inputs_embeds=pt.input_proj(h)).last_hidden_state).permute(0, 2, 1)
            for blocks in self.upsample:
                for b in blocks:
                    h = b(h)
            for b in self.decoder:
                h = b(h)
            return h.clamp(-1, 1)

    o = Oracle()
    for n, p in o.named_parameters():
        if not n.startswith("q."):
            if p.dim() > 1:
                torch.nn.init.normal_(p, 0, 0.08)
            else:
                torch.nn.init.normal_(p, 0.8 if "norm" in n else 0.0, 0.1)
    o = o.float().eval()
    cfg = TokenizerDecoderConfig.from_dict({**hc.to_dict(), "codebook_dim": cd, "latent_dim": L})
    m = Qwen3TTSTokenizerDecoder(cfg, torch.float32, "cpu")
    sd = {k: v for k, v in o.state_dict().items() if not k.startswith("q.")}
    sd.update(o.quantizer_names())
    loaded = m.load_weights(sd.items())
    unused = {k for k in sd if "input_proj" in k and k.startswith("quantizer.")}
    assert loaded == set(sd) - unused, sorted(set(sd) - unused - loaded)
    codes = torch.randint(0, bins, (2, G, 13))
    with torch.no_grad():
        ref, out = o(codes)[:, 0], m.decode(codes)
        assert ref.shape == out.shape == (2, 13 * cfg.total_upsample) and 0.02 < ref.abs().max().item() < 0.99
        assert (ref - out).abs().max().item() < 2e-5
        # chunked decoding with left context: windows equal the oracle run on the same windows
        chunks, start = [], 0
        while start < 13:
            end, ctx = min(13, start + 5), (2 if start - 2 > 0 else start)
            chunks.append(o(codes[..., start - ctx:end])[:, 0, ctx * cfg.total_upsample:])
            start = end
        o2 = m.chunked_decode(codes, 5, 2)
        assert (torch.cat(chunks, -1) - o2).abs().max().item() < 2e-5


def test_mel_filterbank_matches_the_slaney_bank_of_transformers():
    from transformers.audio_utils import mel_filter_bank
    from vllm_omni_b200.models.qwen3_tts.speaker import mel_filterbank_slaney, mel_spectrogram
    ref = mel_filter_bank(num_frequency_bins=513, num_mel_filters=128, min_frequency=0, max_frequency=12000,
                          sampling_rate=24000, norm="slaney", mel_scale="slaney")
    mine = mel_filterbank_slaney(24000, 1024, 128, 0, 12000)
    assert (torch.from_numpy(ref).t().float() - mine).abs().max().item() < 1e-7
    wav = 0.5 * torch.sin(torch.arange(24000) / 24000 * 2 * math.pi * 440)[None]
    mel = mel_spectrogram(wav)
    assert mel.shape == (1, 128, 93)                        # (24000 + 768 - 1024) / 256 + 1 frames
    peak = mel[0, :, 40].argmax().item()
    centre = mine[peak].argmax().item() * 24000 / 1024
    assert abs(centre - 440) < 60


# ----------------------------------------------------------------------------- checkpoint folder through the pipeline
TTS_YAML = """
stage_args:
  - stage_id: 0
    stage_type: llm
    runtime: {devices: "0", max_batch_size: 2}
    engine_args: {model_stage: qwen3_tts, model_arch: Qwen3TTSForConditionalGeneration, worker_type: generation,
                  engine_output_type: audio, device: cpu, dtype: float32,
                  model_overrides: {suppress_tail: 16, assistant_token_id: 510, user_token_id: 509, newline_token_id: 11}}
    final_output: true
    final_output_type: audio
"""


def _decoder_checkpoint_names(dec) -> dict:
    """The decoder's tensors under the names the tokenizer checkpoint uses (fused projections split)."""
    out = {}
    H, Hkv, Dh, Fi = dec.pre_transformer.layers[0].H, dec.pre_transformer.layers[0].Hkv, dec.pre_transformer.layers[0].Dh, dec.c.intermediate_size
    for k, v in dec.state_dict().items():
        p = k.split(".")
        if k == "code_table":
            continue
        if p[0] in ("input_proj", "output_proj"):
            out["pre_transformer." + k] = v
        elif k == "pre_transformer.norm":
            out[k + ".weight"] = v
        elif k.startswith("pre_transformer.layers."):
            base, leaf = ".".join(p[:3]), ".".join(p[3:])
            if leaf == "qkv.weight":
                q, kk, vv = v.split([H * Dh, Hkv * Dh, Hkv * Dh])
                out[base + ".self_attn.q_proj.weight"], out[base + ".self_attn.k_proj.weight"], out[base + ".self_attn.v_proj.weight"] = q, kk, vv
            elif leaf == "o.weight":
                out[base + ".self_attn.o_proj.weight"] = v
            elif leaf == "gate_up.weight":
                out[base + ".mlp.gate_proj.weight"], out[base + ".mlp.up_proj.weight"] = v[:Fi], v[Fi:]
            elif leaf == "down.weight":
                out[base + ".mlp.down_proj.weight"] = v
            elif leaf in ("input_layernorm", "post_attention_layernorm"):
                out[base + "." + leaf + ".weight"] = v
            else:
                out[base + "." + {"attn_scale": "self_attn_layer_scale.scale", "mlp_scale": "mlp_layer_scale.scale"}[leaf]] = v
        else:
            out[k] = v
    return out


@pytest.fixture(scope="module")
def tts_folder(tmp_path_factory):
    """A folder laid out like the published one: ``config.json`` with ``talker_config`` /
    ``speaker_encoder_config``, ``model.safetensors`` with ``talker.*`` / ``speaker_encoder.*`` names and
    ``speech_tokenizer/{config.json, model.safetensors}``."""
    tmp_path = tmp_path_factory.mktemp("qwen3_tts_ckpt")
    import json
    from safetensors.torch import save_file
    from vllm_omni_b200.models.qwen3_tts.tokenizer_12hz import Qwen3TTSTokenizerDecoder
    cfg, oracle, m = _pair(4)
    _init(m.speaker_encoder, 0.2)
    t, p, dc, se = cfg.talker, cfg.code_predictor, cfg.tokenizer_decoder, cfg.speaker_encoder
    hf_cfg = {
        "architectures": ["Qwen3TTSForConditionalGeneration"], "model_type": "qwen3_tts", "tts_model_type": "base",
        "tokenizer_type": "qwen3_tts_tokenizer_12hz", "im_start_token_id": cfg.im_start_token_id,
        "im_end_token_id": cfg.im_end_token_id, "tts_pad_token_id": cfg.tts_pad_token_id, "tts_bos_token_id": cfg.tts_bos_token_id,
        "tts_eos_token_id": cfg.tts_eos_token_id,
        "talker_config": {
            "vocab_size": t.vocab_size, "hidden_size": t.hidden_size, "num_hidden_layers": t.num_hidden_layers,
            "num_attention_heads": t.num_attention_heads, "num_key_value_heads": t.num_key_value_heads, "head_dim": t.head_dim,
            "intermediate_size": t.intermediate_size, "rope_theta": 10000, "rope_scaling": {"mrope_section": [2, 3, 3], "interleaved": True},
            "text_hidden_size": cfg.text_hidden_size, "text_vocab_size": cfg.text_vocab_size, "num_code_groups": p.num_code_groups,
            "codec_eos_token_id": cfg.codec_eos_id, "codec_think_id": cfg.codec_think_id, "codec_nothink_id": cfg.codec_nothink_id,
            "codec_think_bos_id": cfg.codec_think_bos_id, "codec_think_eos_id": cfg.codec_think_eos_id, "codec_pad_id": cfg.codec_pad_id,
            "codec_bos_id": cfg.codec_bos_id, "spk_id": {"Vivian": 80, "Uncle_Fu": 81}, "spk_is_dialect": {"Vivian": False, "Uncle_Fu": "beijing"},
            "codec_language_id": cfg.codec_language_id,
            "code_predictor_config": {"vocab_size": p.vocab_size, "hidden_size": p.hidden_size, "num_hidden_layers": p.num_hidden_layers,
                                      "num_attention_heads": p.num_attention_heads, "num_key_value_heads": p.num_key_value_heads,
                                      "head_dim": p.head_dim, "intermediate_size": p.intermediate_size, "num_code_groups": p.num_code_groups}},
        "speaker_encoder_config": {"mel_dim": se.mel_dim, "enc_dim": se.enc_dim, "enc_channels": list(se.enc_channels),
                                   "enc_kernel_sizes": list(se.enc_kernel_sizes), "enc_dilations": list(se.enc_dilations),
                                   "enc_attention_channels": se.enc_attention_channels, "enc_res2net_scale": se.enc_res2net_scale,
                                   "enc_se_channels": se.enc_se_channels, "sample_rate": 24000}}
    (tmp_path / "config.json").write_text(json.dumps(hf_cfg))
    sd = {k: v.detach().clone().contiguous() for k, v in oracle.checkpoint().items()}
    sd.update({"speaker_encoder." + k: v.detach().clone().contiguous() for k, v in m.speaker_encoder.state_dict().items()})
    save_file(sd, str(tmp_path / "model.safetensors"))
    # the tokenizer folder: a decoder with its own (non-default) geometry under ``decoder.``
    torch.manual_seed(5)
    dec = Qwen3TTSTokenizerDecoder(dc, torch.float32, "cpu")
    with torch.no_grad():
        for n, q in dec.named_parameters():
            q.copy_(torch.randn_like(q) * (0.08 if q.dim() > 1 else 0.1))
    (tmp_path / "speech_tokenizer").mkdir()
    dcd = {k: (list(v) if isinstance(v, tuple) else v) for k, v in dc.__dict__.items()}
    import transformers.models.mimi.modeling_mimi as MM
    mc = MM.MimiConfig(num_filters=4, hidden_size=16, num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=2, head_dim=8,
                       intermediate_size=32, sliding_window=6, codebook_size=dc.codebook_size, codebook_dim=8,
                       vector_quantization_hidden_dimension=8, num_quantizers=6, num_semantic_quantizers=1,
                       upsampling_ratios=[4, 3, 2, 2], frame_rate=250.0, sampling_rate=24000, upsample_groups=16)
    mimi = MM.MimiModel(mc).float().eval()
    (tmp_path / "speech_tokenizer" / "config.json").write_text(json.dumps({
        "model_type": "qwen3_tts_tokenizer_12hz", "decoder_config": dcd, "encoder_config": mc.to_dict(),
        "encoder_valid_num_quantizers": dc.num_quantizers}))
    G, bins, cd = dc.num_quantizers, dc.codebook_size, dc.codebook_dim
    tsd = {"decoder." + k: v.detach().clone().contiguous() for k, v in _decoder_checkpoint_names(dec).items()}
    table = torch.zeros(G, bins, cd)
    for grp, idx in (("rvq_first", [0]), ("rvq_rest", list(range(1, G)))):
        proj = torch.randn(cd, cd // 2, 1) * 0.3
        tsd[f"decoder.quantizer.{grp}.output_proj.weight"] = proj
        for li, g in enumerate(idx):
            s, u = torch.randn(bins, cd // 2), torch.rand(bins) * 2 + 0.5
            tsd[f"decoder.quantizer.{grp}.vq.layers.{li}._codebook.embedding_sum"] = s
            tsd[f"decoder.quantizer.{grp}.vq.layers.{li}._codebook.cluster_usage"] = u
            table[g] = (s / u[:, None]) @ proj[:, :, 0].t()
    tsd.update({"encoder." + k: v.detach().clone().contiguous() for k, v in mimi.state_dict().items()})
    save_file(tsd, str(tmp_path / "speech_tokenizer" / "model.safetensors"))
    with torch.no_grad():
        dec.code_table.copy_(table.view(G * bins, cd))
    (tmp_path / "stages.yaml").write_text(TTS_YAML)

    return tmp_path, cfg, oracle, dec, sd, mimi


def test_checkpoint_folder_through_the_pipeline(tts_folder):
    """Served through ``Omni``: the frames equal the oracle's greedy frames and the waveform equals the
    decoder run on them."""
    from vllm_omni_b200.entrypoints.omni import Omni
    from vllm_omni_b200.entrypoints.stage_runtime import inproc_adapter
    from vllm_omni_b200.inputs import SamplingParams
    tmp_path, cfg, oracle, dec, sd, mimi = tts_folder
    dc = cfg.tokenizer_decoder
    ids = _wrapped(cfg, TEXT)
    with torch.no_grad():
        ro, to, po = oracle.prompt(ids, spk_embed=oracle.codec([80]), language_id=cfg.codec_language_id["english"])
        ref = oracle.generate(ro, to, po, steps=7)
    o = Omni(str(tmp_path), stage_configs_path=str(tmp_path / "stages.yaml"))
    try:
        prompt = {"prompt_token_ids": TEXT, "additional_information": {"task_type": "CustomVoice", "speaker": "Vivian", "language": "English"}}
        outs = o.generate([prompt], [SamplingParams(temperature=0.0, max_tokens=7, seed=1)])
        mm = outs[0].multimodal_output
        assert torch.equal(mm["codes"].cpu(), ref)
        want = dec.chunked_decode(ref.t()[None].contiguous())[0]
        assert mm["audio"].shape == want.shape and (mm["audio"].cpu() - want).abs().max().item() < 1e-5
        live = inproc_adapter(0).llm.model
        assert live.cfg.spk_id == {"vivian": 80, "uncle_fu": 81} and live.cfg.tts_model_type == "base"
        assert torch.equal(live.speaker_encoder.fc.weight, sd["speaker_encoder.fc.weight"])
        # x-vector cloning on the served model: the reference clip rides in the request
        clip = (0.3 * torch.sin(torch.arange(12000) / 24000 * 2 * math.pi * 180)).tolist()
        p2 = {"prompt_token_ids": TEXT, "additional_information": {"task_type": "Base", "ref_audio": clip, "ref_sr": 24000,
                                                                   "x_vector_only_mode": True}}
        outs = o.generate([p2], [SamplingParams(temperature=0.0, max_tokens=4, seed=1)])
        assert outs[0].multimodal_output["audio"].numel() == outs[0].multimodal_output["codes"].shape[0] * dc.total_upsample
        # in-context cloning: the clip's frames come from the tokenizer's own encoder (= transformers' Mimi on the same weights)
        voice = live.create_voice_clone_prompt(torch.tensor(clip), 24000, ref_ids=[41, 42])
        want_code = mimi.encode(torch.tensor(clip)[None, None], num_quantizers=dc.num_quantizers).audio_codes[0].t()
        assert voice["icl_mode"] and torch.equal(voice["ref_code"], want_code[: voice["ref_code"].shape[0]])
        p3 = {"prompt_token_ids": TEXT, "additional_information": {"task_type": "Base", "ref_audio": clip, "ref_sr": 24000,
                                                                   "ref_token_ids": [41, 42]}}
        outs = o.generate([p3], [SamplingParams(temperature=0.0, max_tokens=3, seed=1)])
        assert outs[0].multimodal_output["codes"].shape[1] == dc.num_quantizers and outs[0].multimodal_output["audio"].numel() > 0
    finally:
        o.close()


def test_speech_endpoint_on_a_tts_checkpoint(tts_folder):
    """``/v1/audio/speech`` on the served folder: voices come from the checkpoint's table, a named voice
    and a cloned voice (reference WAV as base64) both return RIFF audio, bad requests are refused."""
    import base64
    pytest.importorskip("fastapi")
    from fastapi.testclient import TestClient
    from vllm_omni_b200.entrypoints.async_omni import AsyncOmni
    from vllm_omni_b200.entrypoints.openai.api_server import build_app
    from vllm_omni_b200.entrypoints.openai.media_utils import wav_bytes
    tmp_path = tts_folder[0]
    eng = AsyncOmni(str(tmp_path), stage_configs_path=str(tmp_path / "stages.yaml"))
    try:
        with TestClient(build_app(eng, "tiny-tts", kind="omni")) as c:
            assert c.get("/v1/audio/voices").json()["voices"] == ["Vivian", "Uncle_Fu"]
            r = c.post("/v1/audio/speech", json={"input": "hello", "voice": "vivian", "language": "English", "max_new_tokens": 4})
            assert r.status_code == 200 and r.content[:4] == b"RIFF", r.text
            clip = 0.3 * torch.sin(torch.arange(12000) / 24000 * 2 * math.pi * 180)
            b64 = base64.b64encode(wav_bytes(clip, 24000)).decode()
            r = c.post("/v1/audio/speech", json={"input": "hello", "ref_audio": b64, "x_vector_only_mode": True, "max_new_tokens": 4})
            assert r.status_code == 200 and r.content[:4] == b"RIFF", r.text
            r = c.post("/v1/audio/speech", json={"input": "hello", "task_type": "VoiceDesign", "instructions": "a calm low voice",
                                                 "max_new_tokens": 4})
            assert r.status_code == 200 and r.content[:4] == b"RIFF", r.text
            assert c.post("/v1/audio/speech", json={"input": "x", "voice": "nobody"}).status_code == 400
            assert c.post("/v1/audio/speech", json={"input": "x", "task_type": "Base"}).status_code == 400
            assert c.post("/v1/audio/speech", json={"input": "x", "task_type": "VoiceDesign"}).status_code == 400
    finally:
        eng.close()


def test_tokenizer_encoder_against_hf_mimi():
    """The 12 Hz tokenizer's encoder is transformers' Mimi analysis path: same frames from the same
    state dict (SEANet stack, sliding-window transformer, stride-2 downsampling, split quantizer)."""
    M = pytest.importorskip("transformers.models.mimi.modeling_mimi")
    from vllm_omni_b200.models.qwen3_tts.tokenizer_12hz_encoder import MimiEncoderConfig, Qwen3TTSTokenizerEncoder
    torch.manual_seed(0)
    hc = M.MimiConfig(num_filters=4, hidden_size=32, num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=2, head_dim=16,
                      intermediate_size=64, sliding_window=6, codebook_size=32, codebook_dim=8, vector_quantization_hidden_dimension=8,
                      num_quantizers=6, num_semantic_quantizers=1, upsampling_ratios=[4, 3, 2, 2], frame_rate=250.0, sampling_rate=24000,
                      upsample_groups=32)
    hf = M.MimiModel(hc).float().eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            p.copy_(torch.randn_like(p) * (0.2 if p.dim() > 1 else 0.1) + (1.0 if "layernorm" in n and n.endswith("weight") else 0.0))
        for n, b in hf.named_buffers():
            if n.endswith("embed_sum"):
                b.copy_(torch.randn_like(b))
            elif n.endswith("cluster_usage"):
                b.copy_(torch.rand_like(b) + 0.5)
    cfg = MimiEncoderConfig.from_dict(hc.to_dict())
    assert cfg.encodec_frame_rate == 500.0
    m = Qwen3TTSTokenizerEncoder(cfg, valid_quantizers=4, device="cpu")
    sd = {k: v for k, v in hf.state_dict().items()
          if k.startswith(("encoder.", "encoder_transformer.", "downsample.", "quantizer.")) and "output_proj" not in k and "initialized" not in k}
    loaded = m.load_weights(sd.items())
    assert loaded == set(sd), sorted(set(sd) - loaded)[:5]
    wav = torch.randn(1, 1, 1000) * 0.3
    with torch.no_grad():
        ref_emb = hf.downsample(hf.encoder_transformer(hf.encoder(wav).transpose(1, 2))[0].transpose(1, 2))
        emb = m.features(wav[:, 0])
        assert ref_emb.shape == emb.shape and (ref_emb - emb).abs().max().item() < 1e-4 * max(1.0, ref_emb.abs().max().item())
        ref = hf.encode(wav, num_quantizers=4).audio_codes[0]                # [K, T']
        got = m.encode(wav[0, 0])
    assert got.shape == (ref.shape[1], 4) and torch.equal(got, ref.t())
