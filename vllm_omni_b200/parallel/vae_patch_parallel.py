"""VAE decode across ranks (K12 / P11).

* ``plan_tiles`` / ``blend_tiles``: overlapping latent tiles with linear cross-fades — the
  tiled decode of a single GPU and the stitch rule of ``_distributed_tiled_decode``
  (vllm_omni/diffusion/distributed/vae_patch_parallel.py:71-205).
* ``VaePatchParallelism``: every rank already holds the full latent (it is tiny), decodes the
  tiles assigned to it round-robin and the RGB tiles are collected on rank 0
  (``_distributed_patch_decode``, :208-345) — on GPUs by peer stores into rank 0's image
  buffer followed by a barrier instead of gather + broadcast.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class Tile:
    y0: int
    y1: int
    x0: int
    x1: int


def plan_tiles(H: int, W: int, tile: int, overlap: int) -> list[Tile]:
    """Latent-space tiles of side ``tile`` that advance by tile - overlap and cover [0,H)x[0,W)."""
    step = max(1, tile - overlap)
    ys = list(range(0, max(H - overlap, 1), step))
    xs = list(range(0, max(W - overlap, 1), step))
    tiles = []
    for y in ys:
        for x in xs:
            y1, x1 = min(H, y + tile), min(W, x + tile)
            tiles.append(Tile(max(0, y1 - tile) if y1 == H and H >= tile else y, y1,
                              max(0, x1 - tile) if x1 == W and W >= tile else x, x1))
    seen, out = set(), []
    for t in tiles:
        k = (t.y0, t.y1, t.x0, t.x1)
        if k not in seen:
            seen.add(k)
            out.append(t)
    return out


def _ramp(n: int, lo: int, hi: int, device) -> torch.Tensor:
    """Weight profile of length n: ramps up over ``lo`` samples, down over ``hi`` samples."""
    w = torch.ones(n, device=device)
    if lo > 0:
        w[:lo] = (torch.arange(lo, device=device) + 1) / (lo + 1)
    if hi > 0:
        w[n - hi:] = torch.minimum(w[n - hi:], (torch.arange(hi, 0, -1, device=device)) / (hi + 1))
    return w


def blend_tiles(decoded: list[tuple[Tile, torch.Tensor]], H: int, W: int, scale: int, overlap_px: int) -> torch.Tensor:
    """Weighted average of decoded tiles (pixel space); weights fade linearly inside overlaps."""
    t0 = decoded[0][1]
    out = torch.zeros(t0.shape[0], t0.shape[1], H, W, dtype=torch.float32, device=t0.device)
    acc = torch.zeros(1, 1, H, W, dtype=torch.float32, device=t0.device)
    for t, img in decoded:
        y0, y1, x0, x1 = t.y0 * scale, t.y1 * scale, t.x0 * scale, t.x1 * scale
        wy = _ramp(y1 - y0, overlap_px if y0 > 0 else 0, overlap_px if y1 < H else 0, img.device)
        wx = _ramp(x1 - x0, overlap_px if x0 > 0 else 0, overlap_px if x1 < W else 0, img.device)
        w = wy[:, None] * wx[None, :]
        out[:, :, y0:y1, x0:x1] += img.float() * w
        acc[:, :, y0:y1, x0:x1] += w
    return (out / acc.clamp_min(1e-6)).to(t0.dtype)


class VaePatchParallelism:
    def __init__(self, pipe, size: int, tile_latent: int = 64, overlap: int = 8):
        self.pipe, self.size = pipe, size
        self.tile, self.overlap = tile_latent, overlap

    def install(self):
        from . import parallel_state as ps
        self.group = ps.get_vae_parallel_group()
        self.pipe.vae_decode = self.decode
        return self

    @torch.no_grad()
    def decode(self, z: torch.Tensor) -> torch.Tensor:
        vae = self.pipe.vae
        g = self.group
        P, r = g.world_size, g.rank_in_group
        B, C, H, W = z.shape
        s = vae.cfg.spatial_scale
        tiles = plan_tiles(H, W, self.tile, self.overlap)
        if P == 1 or len(tiles) == 1:
            return vae.decode(z)
        zz = vae.denormalize(z.float()).to(vae.dtype)
        mine = [(i, t) for i, t in enumerate(tiles) if i % P == r]
        dec = [(i, vae.decoder(vae.post_quant_conv(zz[:, :, t.y0:t.y1, t.x0:t.x1]))) for i, t in mine]
        # collect on rank 0 (tiles differ in size: exchange as objects on CPU groups for the
        # host path, tensors per tile on the device path)
        gathered: list = [None] * len(tiles)
        for i, t in enumerate(tiles):
            owner = i % P
            shape = (B, 3, (t.y1 - t.y0) * s, (t.x1 - t.x0) * s)
            buf = next(d for j, d in dec if j == i) if owner == r else torch.empty(shape, dtype=vae.dtype, device=z.device)
            if owner != 0:
                if r == owner:
                    torch.distributed.send(buf.contiguous(), dst=g.ranks[0], group=g.device_group)
                elif r == 0:
                    torch.distributed.recv(buf, src=g.ranks[owner], group=g.device_group)
            if r == 0:
                gathered[i] = (t, buf)
        if r == 0:
            img = blend_tiles(gathered, H * s, W * s, s, self.overlap * s).clamp_(-1, 1)
        else:
            img = torch.empty(B, 3, H * s, W * s, dtype=vae.dtype, device=z.device)
        g.broadcast(img, src=0)
        return img
