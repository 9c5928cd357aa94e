"""Qwen-Image edit pipelines on CPU: the condition image reaches the denoiser twice, as VAE latents
appended to the token sequence and through the vision-language prompt encoder."""
import re

import torch

from vllm_omni_b200.diffusion.data import OmniDiffusionConfig, TransformerConfig
from vllm_omni_b200.diffusion.models.qwen_image.pipeline_edit import QwenImageEditPipeline, QwenImageEditPlusPipeline
from vllm_omni_b200.diffusion.models.qwen_image.text_encoder import QwenVLTextEncoder
from vllm_omni_b200.diffusion.models.vae.autoencoder_kl_qwenimage import QwenImageVAEConfig
from vllm_omni_b200.diffusion.request import OmniDiffusionRequest
from vllm_omni_b200.inputs import OmniDiffusionSamplingParams
from vllm_omni_b200.models.qwen2_5_vl_vision import Qwen25VisionConfig
from vllm_omni_b200.models.qwen_decoder import DecoderConfig

TF = dict(num_layers=1, attention_head_dim=32, num_attention_heads=2, joint_attention_dim=64, axes_dims_rope=[8, 12, 12])


class SlotTokenizer:
    MARK = {"<|vision_start|>": 290, "<|image_pad|>": 291, "<|vision_end|>": 292}

    def encode(self, text, add_special_tokens=False):
        out = []
        for part in re.split("(" + "|".join(re.escape(k) for k in self.MARK) + ")", text):
            out.extend([self.MARK[part]] if part in self.MARK else list(part.encode()))
        return out


def _pipe(cls):
    torch.manual_seed(0)
    cfg = OmniDiffusionConfig(dtype=torch.float32, tf_model_config=TransformerConfig.from_dict(TF), output_type="latent")
    pipe = cls(cfg, vae_config=QwenImageVAEConfig(base_dim=8, num_res_blocks=1), device="cpu")
    text = DecoderConfig(vocab_size=300, hidden_size=64, intermediate_size=96, num_hidden_layers=1, num_attention_heads=4,
                         num_key_value_heads=2, head_dim=16, qk_norm=False, attention_bias=True, mrope_section=(2, 3, 3))
    vis = Qwen25VisionConfig(depth=2, hidden_size=32, intermediate_size=48, num_heads=2, out_hidden_size=64, patch_size=4,
                             window_size=16, fullatt_block_indexes=(1,))
    pipe.text_encoder = QwenVLTextEncoder(text, SlotTokenizer(), torch.float32, "cpu", vision_config=vis, image_token_id=291)
    return pipe


def _run(pipe, images, seed=3):
    sp = OmniDiffusionSamplingParams(height=64, width=64, num_inference_steps=2, true_cfg_scale=2.0, seed=seed, output_type="latent")
    prompt = {"prompt": "make the sky green", "negative_prompt": "blurry", "multi_modal_data": {"image_tensor": images}}
    return pipe.forward(OmniDiffusionRequest(prompts=[prompt], sampling_params=sp, request_ids=["r"])).output


def test_edit_prompt_states_depend_on_the_condition_image():
    pipe = _pipe(QwenImageEditPipeline)
    pipe.vl_image_area = 48 * 48
    g = torch.Generator().manual_seed(1)
    a, b = torch.rand(3, 40, 56, generator=g), torch.rand(3, 40, 56, generator=g)
    pa, ma = pipe.encode_edit_prompt(["turn left"], [[a]])
    pb, mb = pipe.encode_edit_prompt(["turn left"], [[b]])
    pt, mt = pipe.encode_edit_prompt(["turn left"], [[]])            # no image: text-only path
    assert pa.shape == pb.shape and (pa - pb).abs().max() > 1e-3
    assert int(ma.sum()) > int(mt.sum())                            # the image tokens add prompt rows
    lat_a, lat_b = _run(pipe, [a]), _run(pipe, [b])
    assert lat_a.shape == lat_b.shape == (1, 16, 64) and not torch.equal(lat_a, lat_b)
    assert torch.equal(_run(pipe, [a]), lat_a)                      # deterministic


def test_edit_plus_numbers_its_pictures_and_takes_several():
    pipe = _pipe(QwenImageEditPlusPipeline)
    pipe.vl_image_area = 40 * 40
    seen = []
    orig = pipe.text_encoder.encode_with_images
    pipe.text_encoder.encode_with_images = lambda prompts, images, *a, **k: (seen.append((prompts, [len(r) for r in images])) or
                                                                            orig(prompts, images, *a, **k))
    g = torch.Generator().manual_seed(2)
    imgs = [torch.rand(3, 32, 32, generator=g) for _ in range(2)]
    out = _run(pipe, imgs)
    assert out.shape == (1, 16, 64)
    assert seen[0][1] == [2] and seen[0][0][0].startswith("Picture 1: <|vision_start|>") and "Picture 2: " in seen[0][0][0]
