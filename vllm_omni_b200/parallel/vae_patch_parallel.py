"""VAE decode across ranks (K12 / P11).

* ``plan_tiles`` / ``blend_tiles``: overlapping latent tiles with linear cross-fades — the
  tiled decode of a single GPU and the stitch rule of ``_distributed_tiled_decode``
  (vllm_omni/diffusion/distributed/vae_patch_parallel.py:71-205).
* ``VaePatchParallelism``: every rank already holds the full latent (it is tiny).
  - Latents that need several tiles: each rank decodes the tiles assigned to it round-robin and the
    RGB tiles are blended on rank 0 and broadcast (``_distributed_tiled_decode``).
  - Latents below the tiling threshold: ONE spatial block per rank (a rows x cols grid), decoded with
    a halo of neighbouring latent rows / columns so that the convolutions see their true context,
    cropped back to the core (``_distributed_patch_decode``, :208-345).  The reference pads the
    blocks, gathers them on rank 0, stitches and broadcasts; here every rank stores its core block
    straight into the image buffer of EVERY rank (symmetric peer memory, this library's pitched copy
    kernel) and one bounded-wait barrier ends the exchange, so nothing is gathered or broadcast.
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


def grid_for(n: int) -> tuple[int, int]:
    """rows x cols = n, as square as possible (rows <= cols)."""
    r = int(n ** 0.5)
    while n % r:
        r -= 1
    return r, n // r


def block_bounds(H: int, W: int, rows: int, cols: int, idx: int, halo_base: int):
    """(core h0, h1, w0, w1) and (padded h0, h1, w0, w1) of block ``idx`` of a rows x cols grid over an
    H x W latent; the halo is at least ``halo_base`` and half the core's shorter side."""
    br, bc = idx // cols, idx % cols
    h0, h1 = (br * H) // rows, ((br + 1) * H) // rows
    w0, w1 = (bc * W) // cols, ((bc + 1) * W) // cols
    halo = max(halo_base, min(h1 - h0, w1 - w0) // 2)
    return (h0, h1, w0, w1), (max(0, h0 - halo), min(H, h1 + halo), max(0, w0 - halo), min(W, w1 + halo))


class VaePatchParallelism:
    def __init__(self, pipe, size: int, tile_latent: int = 64, overlap: int = 8):
        self.pipe, self.size = pipe, size
        self.tile, self.overlap = tile_latent, overlap
        self.arena = None
        self._img = None

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
        if P == 1:
            return vae.decode(z)
        if len(tiles) == 1:
            return self._decode_blocks(z)
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

    @torch.no_grad()
    def _decode_blocks(self, z: torch.Tensor) -> torch.Tensor:
        """One core block per rank, decoded with a latent halo and cropped; see the module docstring."""
        vae, g = self.pipe.vae, self.group
        P, r = g.world_size, g.rank_in_group
        B, C, H, W = z.shape
        s = vae.cfg.spatial_scale
        rows, cols = grid_for(P)
        if H < rows or W < cols:
            return vae.decode(z)
        zz = vae.denormalize(z.float()).to(vae.dtype)
        (h0, h1, w0, w1), (ph0, ph1, pw0, pw1) = block_bounds(H, W, rows, cols, r, self.overlap // 2)
        dec = vae.decoder(vae.post_quant_conv(zz[:, :, ph0:ph1, pw0:pw1]))
        core = dec[:, :, (h0 - ph0) * s:(h1 - ph0) * s, (w0 - pw0) * s:(w1 - pw0) * s].clamp(-1, 1).contiguous()
        Hs, Ws = H * s, W * s
        es = core.element_size()
        if z.is_cuda and (w0 * s * es) % 16 == 0 and (core.shape[-1] * es) % 16 == 0 and (Ws * es) % 16 == 0:
            import ctypes
            from ..ops import _native as nv
            from .peer_memory import PeerArena
            key = (B, core.shape[1], Hs, Ws, core.dtype)
            if self._img is None or self._key != key:
                if self.arena is not None:
                    self.arena.close()
                self._key = key
                self.arena = PeerArena(g, B * core.shape[1] * Hs * Ws * es + 8192, z.device)
                self._img = self.arena.alloc((B, core.shape[1], Hs, Ws), core.dtype)
            self.arena.barrier()                    # the previous image has been consumed everywhere
            lib = nv.lib("peer_rt")
            ch, cw = core.shape[-2], core.shape[-1]
            planes = core.view(B * core.shape[1], ch, cw)
            for d in range(P):                      # my block into every rank's image, plane by plane
                for pl in range(planes.shape[0]):
                    dst = self._img.ptrs[d] + ((pl * Hs + h0 * s) * Ws + w0 * s) * es
                    nv.check_rc(lib.omni_peer_copy_2d(ctypes.c_void_p(dst), ctypes.c_size_t(Ws * es), nv.ptr(planes[pl]),
                                                      ctypes.c_size_t(cw * es), ctypes.c_size_t(cw * es), ctypes.c_long(ch),
                                                      nv.stream_ptr()), "omni_peer_copy_2d")
            self.arena.barrier()                    # every block has landed
            return self._img.local.clone()
        # host path (Gloo) and odd geometries: padded blocks, all-gather, stitch everywhere
        mh, mw = -(-H // rows) * s + s, -(-W // cols) * s + s
        pad = torch.zeros(B, core.shape[1], mh, mw, dtype=core.dtype, device=z.device)
        pad[:, :, :core.shape[-2], :core.shape[-1]] = core
        blocks = g.all_gather(pad, separate_tensors=True)
        img = torch.empty(B, core.shape[1], Hs, Ws, dtype=core.dtype, device=z.device)
        for i in range(P):
            (a0, a1, b0, b1), _ = block_bounds(H, W, rows, cols, i, self.overlap // 2)
            img[:, :, a0 * s:a1 * s, b0 * s:b1 * s] = blocks[i][:, :, :(a1 - a0) * s, :(b1 - b0) * s]
        return img

    def close(self):
        if self.arena is not None:
            self.arena.close()
            self.arena = None
