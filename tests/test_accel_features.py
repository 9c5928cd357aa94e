"""Acceleration features around the DiT on CPU: fp8 block-scaled quantisation of a pipeline's
linear layers, LoRA adapters (load from a PEFT directory, activate, LRU / pin, remove), platform
and plugin plumbing, CLI flag mapping."""
import json
import types

import pytest
import torch

from vllm_omni_b200.diffusion.models.qwen_image.transformer import (QwenImageTransformer2DModel,
                                                                    QwenImageTransformerConfig)


def _tiny(dim_heads=4, head_dim=32):
    cfg = QwenImageTransformerConfig(num_layers=2, attention_head_dim=head_dim, num_attention_heads=dim_heads,
                                     joint_attention_dim=64, in_channels=16, out_channels=4, axes_dims_rope=(8, 12, 12))
    torch.manual_seed(0)
    m = QwenImageTransformer2DModel(cfg, dtype=torch.float32, device="cpu")
    for p in m.parameters():
        if p.dim() > 1:
            p.data.normal_(0, 0.05)
    return m


def _run(m):
    g = torch.Generator().manual_seed(1)
    x = torch.randn(1, 64, 16, generator=g)
    e = torch.randn(1, 6, 64, generator=g)
    return m(x, e, torch.tensor([0.5]), (1, 8, 8))


def test_fp8_quantize_pipeline_cpu():
    from vllm_omni_b200.diffusion.quantization.fp8 import DiffusionFp8Config, quantize_pipeline
    m = _tiny()
    ref = _run(m)
    pipe = types.SimpleNamespace(transformer=m)
    od = types.SimpleNamespace(quantization="fp8",
                               quantization_config=DiffusionFp8Config(min_features=128, ignored_layers=["*txt.mlp_*"]))
    n = quantize_pipeline(pipe, od)
    blk = m.blocks[0]
    assert n > 0 and blk.img.to_qkv.fp8 is not None and blk.img.to_qkv.weight.numel() == 0
    assert blk.txt.mlp_up.fp8 is None and blk.txt.mlp_up.weight.numel() > 0          # ignored by pattern
    assert m.proj_out.fp8 is None                                                     # small / excluded layers stay
    out = _run(m)
    rel = (out - ref).norm() / ref.norm()
    assert rel < 0.08, rel
    with pytest.raises(ValueError):
        DiffusionFp8Config.from_dict({"weight_block_size": [64, 64]})


def _write_adapter(tmp_path, m, rank=4, seed=0):
    from vllm_omni_b200.utils.safetensors_reader import save_safetensors
    g = torch.Generator().manual_seed(seed)
    D = m.cfg.inner_dim
    tensors = {}
    for mod, (din, dout) in {"blocks.0.img.to_out": (D, D), "blocks.1.img.mlp_up": (D, m.cfg.mlp_ratio * D)}.items():
        tensors[f"base_model.model.{mod}.lora_A.weight"] = torch.randn(rank, din, generator=g) * 0.1
        tensors[f"base_model.model.{mod}.lora_B.weight"] = torch.randn(dout, rank, generator=g) * 0.1
    d = tmp_path / f"adapter{seed}"
    d.mkdir()
    save_safetensors(tensors, str(d / "adapter_model.safetensors"))
    (d / "adapter_config.json").write_text(json.dumps({"r": rank, "lora_alpha": 2 * rank}))
    return str(d), tensors


def test_lora_manager_activate_lru_pin_remove(tmp_path):
    from vllm_omni_b200.diffusion.lora.manager import DiffusionLoRAManager
    m = _tiny()
    base = _run(m)
    mgr = DiffusionLoRAManager(types.SimpleNamespace(transformer=m), max_cached=2)
    path, tensors = _write_adapter(tmp_path, m)
    lid = mgr.add_adapter_from_path("style", path)
    assert mgr.list_adapters() == [lid]
    mgr.set_active(["style"])
    out = _run(m)
    assert (out - base).abs().max() > 1e-4
    # the delta is exactly scale * B A x on the adapted layer: check it on one module in isolation
    lin = m.blocks[0].img.to_out
    x = torch.randn(3, lin.in_features)
    A, B = tensors["base_model.model.blocks.0.img.to_out.lora_A.weight"], tensors["base_model.model.blocks.0.img.to_out.lora_B.weight"]
    want = torch.nn.functional.linear(x, lin.weight, lin.bias) + 2.0 * (x @ A.t()) @ B.t()
    assert torch.allclose(lin(x), want, atol=1e-4)
    mgr.set_active([])
    assert torch.allclose(_run(m), base, atol=1e-6)
    # LRU with pinning: the pinned adapter survives two further loads
    mgr.pin_adapter(lid)
    ids = [mgr.add_adapter_from_path(f"a{s}", _write_adapter(tmp_path, m, seed=s)[0]) for s in (1, 2)]
    assert lid in mgr.list_adapters() and len(mgr.list_adapters()) == 2 and ids[1] in mgr.list_adapters()
    assert mgr.remove_adapter(lid) and lid not in mgr.list_adapters()
    with pytest.raises(KeyError):
        mgr.set_active(["style"])


def test_platform_and_plugins():
    from vllm_omni_b200 import platforms, plugins
    p = platforms.current_platform() if hasattr(platforms, "current_platform") else platforms.CpuPlatform
    assert hasattr(p, "is_available") and hasattr(p, "device_count")
    assert isinstance(plugins.load_plugins_by_group("vllm_omni.general_plugins"), dict)
    plugins.load_general_plugins()


def test_cli_serve_flags_map_to_engine_kwargs():
    import argparse
    from vllm_omni_b200.entrypoints.cli import main as cli
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd")
    cli.make_serve_parser(sub)
    a = ap.parse_args(["serve", "Qwen/Qwen-Image", "--ulysses-degree", "4", "--cfg-parallel-size", "2", "--cache-backend",
                       "tea_cache", "--port", "9000"])
    kw = cli.serve_kwargs(a)
    pc = kw["parallel_config"]
    assert (pc.ulysses_degree, pc.cfg_parallel_size) == (4, 2) and kw["cache_backend"] == "tea_cache" and a.port == 9000
