"""A diffusers-layout Qwen-Image directory on disk (model_index.json, transformer/ with diffusers
parameter names, text_encoder/ saved by transformers, tokenizer/) served through ``Omni``: the
loader stacks q/k/v and the modulation layers, attaches the Qwen2.5-VL prompt encoder, and the
latents equal those of a pipeline that was handed the same tensors in memory."""
import json

import pytest
import torch

transformers = pytest.importorskip("transformers")
tokenizers = pytest.importorskip("tokenizers")

from vllm_omni_b200.diffusion.data import OmniDiffusionConfig, TransformerConfig
from vllm_omni_b200.diffusion.models.qwen_image.pipeline import QwenImagePipeline
from vllm_omni_b200.diffusion.models.qwen_image.text_encoder import QwenVLTextEncoder, text_config_from_hf
from vllm_omni_b200.entrypoints.omni import Omni
from vllm_omni_b200.inputs import OmniDiffusionSamplingParams
from vllm_omni_b200.utils.safetensors_reader import save_safetensors

TF = dict(num_layers=2, attention_head_dim=32, num_attention_heads=4, joint_attention_dim=64, axes_dims_rope=[8, 12, 12])


def _tokenizer_dir(path):
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers
    alpha = pre_tokenizers.ByteLevel.alphabet()
    tok = Tokenizer(models.BPE(vocab={c: i for i, c in enumerate(sorted(alpha))}, merges=[]))
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = decoders.ByteLevel()
    fast = transformers.PreTrainedTokenizerFast(tokenizer_object=tok, additional_special_tokens=["<|im_start|>", "<|im_end|>"])
    fast.save_pretrained(str(path))


@pytest.fixture(scope="module")
def model_dir(tmp_path_factory):
    d = tmp_path_factory.mktemp("qwen_image_dir")
    torch.manual_seed(0)
    (d / "model_index.json").write_text(json.dumps({"_class_name": "QwenImagePipeline", "_diffusers_version": "0.35.0"}))
    # transformer: random tensors under diffusers names, shapes taken from the name map of a tiny model
    src = QwenImagePipeline(OmniDiffusionConfig(dtype=torch.float32, tf_model_config=TransformerConfig.from_dict(TF)), device="cpu")
    params = dict(src.transformer.named_parameters())
    tensors = {}
    for name, (pn, sl) in src.transformer.checkpoint_name_map().items():
        shape = list(params[pn].shape)
        if sl is not None:
            shape[0] = sl[1] - sl[0]
        tensors[name] = torch.randn(shape) * (0.05 if len(shape) > 1 else 0.2) + (1.0 if "norm" in name and "linear" not in name else 0.0)
    (d / "transformer").mkdir()
    (d / "transformer" / "config.json").write_text(json.dumps({"_class_name": "QwenImageTransformer2DModel", **TF}))
    save_safetensors(tensors, str(d / "transformer" / "diffusion_pytorch_model.safetensors"))
    # text encoder: a tiny HF Qwen2.5-VL saved by transformers
    hc = transformers.Qwen2_5_VLConfig(
        text_config=dict(vocab_size=300, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, max_position_embeddings=2048,
                         rope_parameters=dict(rope_theta=1e6, rope_type="default", mrope_section=[2, 3, 3])),
        vision_config=dict(depth=1, hidden_size=32, intermediate_size=64, num_heads=2, out_hidden_size=64, patch_size=4,
                           fullatt_block_indexes=[0]))
    hf = transformers.Qwen2_5_VLForConditionalGeneration(hc).float().eval()
    hf.save_pretrained(str(d / "text_encoder"))
    _tokenizer_dir(d / "tokenizer")
    return d, tensors, hf, hc


def test_directory_checkpoint_matches_in_memory_weights(model_dir):
    d, tensors, hf, hc = model_dir
    sp = lambda: OmniDiffusionSamplingParams(height=64, width=64, num_inference_steps=2, true_cfg_scale=3.0, seed=5,
                                             output_type="latent")
    prompt = [{"prompt": "a red cube on a table", "negative_prompt": "blurry"}]
    o = Omni(str(d), dtype="float32", device="cpu", output_type="latent")
    try:
        out = o.generate(prompt, sp())[0]
        lat = out.latents if out.latents is not None else torch.as_tensor(out.images[0])
    finally:
        o.close()
    # the same tensors handed over in memory
    ref = QwenImagePipeline(OmniDiffusionConfig(dtype=torch.float32, tf_model_config=TransformerConfig.from_dict(TF),
                                                output_type="latent"), device="cpu")
    assert ref.transformer.load_weights(tensors.items()) == set(tensors)
    enc = QwenVLTextEncoder(text_config_from_hf(hc.to_dict()), transformers.AutoTokenizer.from_pretrained(str(d / "tokenizer")),
                            torch.float32, "cpu")
    enc.load_weights(hf.state_dict().items())
    ref.text_encoder = enc
    from vllm_omni_b200.diffusion.request import OmniDiffusionRequest
    want = ref.forward(OmniDiffusionRequest(prompts=prompt, sampling_params=sp(), request_ids=["r"])).output
    want = want.reshape(lat.shape)
    assert (lat.float() - want.float()).abs().max().item() < 1e-4 and want.abs().max().item() > 0.1
    # and the text encoder really is the checkpoint's: its states differ from the stand-in's
    st, mask = enc(["a red cube on a table"])
    assert st.shape[-1] == 64 and int(mask.sum()) > 0
