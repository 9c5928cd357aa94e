"""Multimodal rotary position ids (vllm_omni/model_executor/layers/rotary_embedding/mrope.py:
24-554): every token gets a (temporal, height, width) triple.  Text tokens advance all three
together; an image/video placeholder run of t*h*w tokens gets its grid coordinates offset by
the running position; an audio run advances like text.  After a multimodal run the next
position is max(previous positions) + 1."""
from __future__ import annotations

import torch


def get_input_positions(input_ids: list[int], image_token_id: int, video_token_id: int, audio_token_id: int,
                        image_grids: list[tuple] | None = None, video_grids: list[tuple] | None = None,
                        seconds_per_grid_t: float = 1.0, position_id_per_seconds: int = 25):
    """Returns (positions int64 [3, L], next_position_delta) where delta = next_pos - L."""
    image_grids = list(image_grids or [])
    video_grids = list(video_grids or [])
    L = len(input_ids)
    pos = torch.zeros(3, L, dtype=torch.long)
    cur = 0
    i = 0
    while i < L:
        tok = input_ids[i]
        if tok in (image_token_id, video_token_id) and (image_grids if tok == image_token_id else video_grids):
            grids = image_grids if tok == image_token_id else video_grids
            t, h, w = grids.pop(0)
            n = t * h * w
            n = min(n, L - i)
            tt = torch.arange(t).repeat_interleave(h * w)
            if tok == video_token_id:
                tt = (tt.float() * seconds_per_grid_t * position_id_per_seconds).long()
            hh = torch.arange(h).repeat_interleave(w).repeat(t)
            ww = torch.arange(w).repeat(t * h)
            pos[0, i:i + n] = cur + tt[:n]
            pos[1, i:i + n] = cur + hh[:n]
            pos[2, i:i + n] = cur + ww[:n]
            cur = int(pos[:, i:i + n].max()) + 1
            i += n
        else:
            pos[:, i] = cur
            cur += 1
            i += 1
    return pos, cur - L


class OmniMRotaryEmbedding:
    """Namespace kept for API parity with the reference class."""
    get_input_positions_tensor = staticmethod(get_input_positions)
