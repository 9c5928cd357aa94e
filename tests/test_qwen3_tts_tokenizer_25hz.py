"""Qwen3-TTS 25 Hz speech tokenizer: Whisper features against the transformers extractor, windowed encoder
attention against a per-window loop, nearest-code search, Euler flow decode, checkpoint names."""
import pytest
import torch
import torch.nn.functional as F

from vllm_omni_b200.models.qwen3_tts.tokenizer_25hz import (Qwen3TTSTokenizer25Hz, Tokenizer25HzConfig,
                                                            build_speech_tokenizer, frames_after_cnn, peak_normalize,
                                                            reference_mel_16k, whisper_log_mel)


def test_whisper_features_match_transformers_extractor():
    from transformers import WhisperFeatureExtractor
    torch.manual_seed(0)
    wav = torch.randn(16000 * 2) * 0.1
    fe = WhisperFeatureExtractor(feature_size=128, sampling_rate=16000, hop_length=160, n_fft=400, chunk_length=2)
    want = fe(wav.numpy(), sampling_rate=16000, return_tensors="pt", padding="max_length").input_features[0]
    got = whisper_log_mel(wav, 128)
    assert got.shape == want.shape == (128, 200)
    assert (got - want).abs().max() < 2e-3


def test_frames_after_cnn():
    conv1, conv2 = torch.nn.Conv1d(4, 4, 3, padding=1), torch.nn.Conv1d(4, 4, 3, stride=2, padding=1)
    for t in (1, 2, 7, 16, 200, 201):
        assert conv2(conv1(torch.zeros(1, 4, t))).shape[-1] == frames_after_cnn(t)


def _tiny(seed=0):
    torch.manual_seed(seed)
    m = Qwen3TTSTokenizer25Hz(Tokenizer25HzConfig.tiny())
    m.encoder.codebook.normal_()
    for p in m.parameters():
        if p.dim() > 1:
            p.normal_(0, 0.2)
    return m


def test_encoder_windows_do_not_mix_and_ragged_path_matches_loop():
    m = _tiny()
    enc, c = m.encoder, m.cfg.encoder
    torch.manual_seed(1)
    # 16 + 16 + 4 mel frames -> windows of 8, 8 and 2 positions: the ragged (masked) path
    mel = torch.randn(c.n_mels, 36)
    got = enc.mel_to_codes([mel])[0]
    # loop reference: each window alone through the blocks, then the joint down-sampling conv
    hs = []
    for part in mel.split(c.n_window * 2, dim=1):
        h = F.gelu(enc.conv2(F.gelu(enc.conv1(part[None]))))[0].T
        h = h + enc.positional_embedding[: h.shape[0]]
        for blk in enc.blocks:
            h = blk(h, [h.shape[0]])
        hs.append(h)
    x = enc.audio_vq_downsample(torch.cat(hs).T[None])[0].T
    want = torch.cdist(x, enc.codebook).argmin(-1)
    assert got.shape == (9,)
    assert torch.equal(got, want)
    # two clips in one call give the same codes as each alone
    mel2 = torch.randn(c.n_mels, 16)
    both = enc.mel_to_codes([mel, mel2])
    assert torch.equal(both[0], got) and torch.equal(both[1], enc.mel_to_codes([mel2])[0])


def test_encode_returns_one_code_per_640_samples_and_unit_xvector():
    m = _tiny()
    m.set_xvector_extractor(lambda w: torch.arange(1.0, 9.0))
    codes, xv, mels = m.encode([torch.randn(6400), torch.randn(24000 // 2)], sr=16000)
    assert [len(c) for c in codes] == [10, 19]            # ceil(12000 / 640) = 19
    assert abs(float(xv[0].norm()) - 1.0) < 1e-6
    assert mels[0].shape == (40, 80)
    # a 24 kHz clip is resampled to 16 kHz before the features
    c24, _, _ = m.encode([torch.randn(24000)], sr=24000)
    assert len(c24[0]) == 25


def test_peak_normalize_and_reference_mel():
    w = torch.randn(4000) * 3
    n = peak_normalize(w)
    assert abs(float(n.abs().max()) - 10 ** (-6 / 20)) < 1e-6
    assert reference_mel_16k(n).shape == (25, 80)


def test_decode_is_euler_flow_then_vocoder_and_trims_padding():
    m = _tiny()
    c = m.cfg
    codes = torch.tensor([[3, 7, 1, 9, 2, 4], [5, 6, 0, 0, 0, 0]])
    xv, ref = torch.randn(2, c.dit.enc_emb_dim), torch.randn(2, 12, c.dit.mel_dim)
    noise = torch.randn(2, 6 * c.dit.repeats, c.dit.mel_dim)
    wavs = m.decode(codes, xv, ref, num_steps=4, noise=noise)
    assert [len(w) for w in wavs] == [6 * c.decode_upsample_rate, 2 * c.decode_upsample_rate]
    # the same integration written out
    from vllm_omni_b200.models.qwen2_5_omni.token2wav import sway_time_grid
    t = sway_time_grid(4, -1.0, "cpu")
    x = noise.clone()
    xvt = xv[:, None].expand(-1, x.shape[1], -1)
    for t0, t1 in zip(t[:-1], t[1:]):
        cond, null = m.dit(x, ref, xvt, codes, t0, apply_cfg=True).chunk(2)
        x = x + (cond + (cond - null) * 0.5) * (t1 - t0)
    want = m.bigvgan(x.transpose(1, 2)).reshape(2, -1)
    assert torch.allclose(wavs[0], want[0][: len(wavs[0])], atol=1e-5)


def test_checkpoint_names_round_trip():
    a, b = _tiny(0), _tiny(1)
    sd = {}
    for n, p in a.encoder.named_parameters():
        sd["encoder.tokenizer." + n] = p.clone()
    sd["encoder.tokenizer.audio_quantizer.rvqs.0.embed"] = a.encoder.codebook.clone()[None]
    sd["encoder.tokenizer.audio_quantizer.rvqs.0.cluster_size"] = torch.zeros(1, 64)     # training state: ignored
    for n, p in a.dit.named_parameters():
        sd["decoder.dit." + n] = p.clone()
    for n, p in a.bigvgan.named_parameters():
        sd["decoder.bigvgan." + n] = p.clone()
    got = b.load_weights(sd.items())
    assert len(got) == len(sd) - 1
    mel = torch.randn(a.cfg.encoder.n_mels, 32)
    assert torch.equal(a.encoder.mel_to_codes([mel])[0], b.encoder.mel_to_codes([mel])[0])


def test_builder_picks_the_class_by_model_type():
    tiny = Tokenizer25HzConfig.tiny()
    cfg = {"model_type": "qwen3_tts_tokenizer_25hz",
           "encoder_config": {k: getattr(tiny.encoder, k) for k in tiny.encoder.__dataclass_fields__},
           "decoder_config": {"dit_config": {k: getattr(tiny.dit, k) for k in tiny.dit.__dataclass_fields__},
                              "bigvgan_config": {k: getattr(tiny.bigvgan, k) for k in tiny.bigvgan.__dataclass_fields__}},
           "decode_upsample_rate": 8}
    m = build_speech_tokenizer(cfg, with_encoder=False)
    assert isinstance(m, Qwen3TTSTokenizer25Hz) and m.encoder is None and m.cfg.decode_upsample_rate == 8
    with pytest.raises(ValueError):
        build_speech_tokenizer({"model_type": "nope"})


def test_stage_model_loads_and_uses_the_25hz_tokenizer(tmp_path):
    """A ``speech_tokenizer/`` folder whose config names the 25 Hz type replaces the 12 Hz decoder on the
    stage model: frames' first column is decoded with the voice's tokenizer x-vector and reference mel."""
    import json

    from safetensors.torch import save_file

    from vllm_omni_b200.models.qwen3_tts.model import Qwen3TTSConfig, Qwen3TTSModel
    src = _tiny(3)
    tiny = src.cfg
    folder = tmp_path / "speech_tokenizer"
    folder.mkdir()
    lst = lambda d: {k: (list(map(list, v)) if v and isinstance(v, tuple) and isinstance(v[0], tuple) else
                         list(v) if isinstance(v, tuple) else v) for k, v in d.items()}
    (folder / "config.json").write_text(json.dumps({
        "model_type": "qwen3_tts_tokenizer_25hz",
        "encoder_config": lst(tiny.encoder.__dict__),
        "decoder_config": {"dit_config": lst(tiny.dit.__dict__), "bigvgan_config": lst(tiny.bigvgan.__dict__)},
        "decode_upsample_rate": tiny.decode_upsample_rate}))
    sd = {"encoder.tokenizer." + n: p.clone() for n, p in src.encoder.named_parameters()}
    sd["encoder.tokenizer.audio_quantizer.rvqs.0.embed"] = src.encoder.codebook.clone()[None]
    sd.update({"decoder.dit." + n: p.clone() for n, p in src.dit.named_parameters()})
    sd.update({"decoder.bigvgan." + n: p.clone() for n, p in src.bigvgan.named_parameters()})
    save_file({k: v.contiguous() for k, v in sd.items()}, str(folder / "model.safetensors"))
    m = Qwen3TTSModel(Qwen3TTSConfig.tiny(), torch.float32, "cpu")
    assert m.load_auxiliary(str(tmp_path)) == len(sd)
    assert m.tokenizer_25hz is not None
    clip = 0.3 * torch.sin(torch.arange(6400) / 16000 * 2 * 3.14159 * 200)
    voice = m.create_voice_clone_prompt(clip, 16000, x_vector_only_mode=True)
    assert voice["ref_mel"].shape == (40, 80) if tiny.dit.mel_dim == 80 else voice["ref_mel"].shape[0] == 40
    frames = torch.tensor([[3], [9], [1], [4]])
    # the tiny flow model takes 8 mel bins: hand it a reference of that width
    v = {"tokenizer_xvector": torch.zeros(tiny.dit.enc_emb_dim), "ref_mel": torch.zeros(12, tiny.dit.mel_dim)}
    wav = m.decode_codes(frames, v)
    want = src.decode(frames[:, 0][None], v["tokenizer_xvector"][None], v["ref_mel"][None])[0]
    assert wav.shape == (4 * tiny.decode_upsample_rate,) and torch.allclose(wav, want, atol=1e-6)
