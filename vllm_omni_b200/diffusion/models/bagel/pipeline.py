"""Bagel image generation stage (vllm_omni/diffusion/models/bagel/pipeline_bagel.py:319-327):
the DiT stage of an AR -> DiT pipeline.  The upstream AR stage prefills the prompt and hands its
KV cache over through the KV transfer manager; this stage injects it as ``past_key_values`` —
every attention layer attends to [received KV | its own tokens] — instead of re-encoding the
prompt."""
from __future__ import annotations

from ..z_image.pipeline import ZImagePipeline
from ..z_image.transformer import ZImageTransformerConfig


class BagelPipeline(ZImagePipeline):
    def __init__(self, od_config=None, transformer_config=None, vae_config=None, device=None, **kw):
        tc = transformer_config or ZImageTransformerConfig.from_dict(od_config.tf_model_config.to_dict() if od_config else {})
        super().__init__(od_config, tc, vae_config, device)

    def forward(self, req):
        sp = req.sampling_params
        if sp.need_kv_receive and sp.past_key_values is None:
            raise RuntimeError("BagelPipeline expects the prompt KV cache from the AR stage (past_key_values); "
                               "none was received")
        return super().forward(req)
