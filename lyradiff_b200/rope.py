"""Rotary-embedding table for the FLUX block ops (host side, runs once per image size).

The block classes take `rope_emb` as a [B, 1, S, head_dim/2, 2, 2] fp32 table whose last two axes hold the rotation
matrix [[cos, -sin], [sin, cos]] of each frequency; `lyraq_rmsnorm_rope` reads it in exactly that layout.  This is the
table the reference's Python wrapper builds before calling the ops (`rope` / `EmbedND`,
lyradiff/lyradiff_model/lyradiff_flux_transformer_model_v2.py:35-65): angles in float64, one block of frequencies per
position axis, concatenated along the frequency axis.
"""

import torch


def axis_table(pos, dim, theta):
    """pos [B, S] -> [B, S, dim/2, 2, 2] fp32 for one position axis with `dim` channels."""
    if dim % 2:
        raise ValueError("rope: the axis dimension must be even, got %d" % dim)
    freq = torch.pow(torch.tensor(float(theta), dtype=torch.float64, device=pos.device),
                     -torch.arange(0, dim, 2, dtype=torch.float64, device=pos.device) / dim)
    ang = pos.to(torch.float64).unsqueeze(-1) * freq
    c, s = torch.cos(ang), torch.sin(ang)
    rot = torch.stack([c, -s, s, c], dim=-1)
    return rot.reshape(pos.shape[0], -1, dim // 2, 2, 2).float()


def flux_rope_table(ids, axes_dim=(16, 56, 56), theta=10000):
    """ids [B, S, n_axes] (text rows all zero, image rows (0, y, x)) -> [B, 1, S, sum(axes_dim)/2, 2, 2] fp32."""
    if ids.shape[-1] != len(axes_dim):
        raise ValueError("rope: ids has %d axes, axes_dim %d" % (ids.shape[-1], len(axes_dim)))
    parts = [axis_table(ids[..., a], axes_dim[a], theta) for a in range(len(axes_dim))]
    return torch.cat(parts, dim=-3).unsqueeze(1)


def flux_position_ids(text_tokens, height, width, batch=1, device="cpu"):
    """Position ids of a FLUX sequence: `text_tokens` zero rows, then height x width image rows (0, y, x)."""
    ids = torch.zeros(batch, text_tokens + height * width, 3, device=device)
    ids[:, text_tokens:, 1] = torch.arange(height, device=device).repeat_interleave(width).float()
    ids[:, text_tokens:, 2] = torch.arange(width, device=device).repeat(height).float()
    return ids
