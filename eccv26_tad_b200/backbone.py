"""Plain-torch restatement of the forward of ``VisionTransformerSparseAdapterPOGUISE`` on top of the
SparseConv2D op and the CUDA table builder (the first "next" row after the hot path itself).

Follows ``opentad/models/backbones/vit_sparse_adapter_poguise.py`` of pcr-upm/eccv26_tad:
patch embedding and fixed sinusoid positions, CLS token, pre-norm blocks whose attention also returns
CLS-attention scores for top-k token selection (``KTPAttention``, :707-789), gather of the kept tokens
and update of the neighbor table (``Block._inner_forward``, :899-977), MLP, and the adapter
``down_proj -> GELU -> SparseConv2d on the patch tokens -> up_proj``, ``x * gamma + input``
(``EfficientAdapter.forward``, :288-362 and :652-653), final norm and frame-mean pooling
(:1762-1838).  mmcv's ``PatchEmbed`` / ``FFN`` / ``DropPath`` and mmaction's sinusoid table are third
party and absent here; the few lines they amount to at inference are written out locally.  Options of
the reference that do not touch the op (heat-map tokens, adapter attention variants, drop path,
activation checkpointing) are left out.

``conv_impl`` selects how the adapters convolve:
  "svtad"  SparseConv2d of this package on the running neighbor table (the product path);
  "dense"  the reference's own ``2d_conv`` branch restated - scatter the kept tokens to the full
           grid, ``F.conv2d``, gather them back (:364-412, :484-490) - with the SAME weights.  It is the
           model-level check of the sparse path and needs no table.
``table_impl`` selects who maintains the table: "svtad" (CUDA kernels) or "torch" (the reference's
tensor ops restated, for checking).
"""

import torch
import torch.nn as nn
import torch.nn.functional as F

from .neighbor_table import get_initial_neighbor_indices, num_keep_tokens, select_and_update, select_topk
from .sparse_conv_layer import SparseConv2d


def sinusoid_table(n_pos, dim):
    """Fixed sine / cosine position table ``[1, n_pos, dim]`` (even channels sin, odd channels cos)."""
    pos = torch.arange(n_pos, dtype=torch.float64).unsqueeze(1)
    i = torch.arange(dim, dtype=torch.float64).unsqueeze(0)
    angle = pos / torch.pow(torch.tensor(10000.0, dtype=torch.float64), 2 * torch.div(i, 2, rounding_mode="floor") / dim)
    table = torch.where((torch.arange(dim) % 2 == 0).unsqueeze(0), torch.sin(angle), torch.cos(angle))
    return table.float().unsqueeze(0)


class KTPAttention(nn.Module):
    """Attention that also scores the patch tokens by the CLS query (reference :656-789)."""

    def __init__(self, dim, num_heads, keep_rate=1.0):
        super().__init__()
        self.num_heads = num_heads
        self.scale = (dim // num_heads) ** -0.5
        self.qkv = nn.Linear(dim, dim * 3, bias=False)
        self.q_bias = nn.Parameter(torch.zeros(dim))
        self.v_bias = nn.Parameter(torch.zeros(dim))
        self.proj = nn.Linear(dim, dim)
        self.keep_rate = keep_rate

    def forward(self, x):
        B, N, C = x.shape
        bias = torch.cat((self.q_bias, torch.zeros_like(self.v_bias), self.v_bias))
        qkv = F.linear(x, self.qkv.weight, bias).reshape(B, N, 3, self.num_heads, -1).permute(2, 0, 3, 1, 4)
        q, k, v = qkv[0], qkv[1], qkv[2]
        out = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B, N, -1)
        out = self.proj(out)
        if self.keep_rate >= 1:
            return out, None
        # CLS query against all keys, softmax, summed over the (single) key token, mean over heads (:743-777)
        attn = ((q[:, :, :1] * self.scale) @ k.transpose(-2, -1)).softmax(dim=-1)
        scores = attn.sum(dim=-2).mean(dim=1)[:, 1:].float()
        return out, scores


class SparseAdapter(nn.Module):
    """``down_proj -> GELU -> 3x3 conv on the patch tokens -> up_proj``, ``x * gamma + input``."""

    def __init__(self, dim, hidden, kernel_size=3):
        super().__init__()
        self.down_proj = nn.Linear(dim, hidden)
        self.act = nn.GELU()
        self.sparse_conv = SparseConv2d(hidden, hidden, kernel_size=kernel_size)
        self.up_proj = nn.Linear(hidden, dim)
        self.gamma = nn.Parameter(torch.ones(1))
        self.kernel_size = kernel_size
        nn.init.trunc_normal_(self.down_proj.weight, std=0.02)
        nn.init.zeros_(self.down_proj.bias)

    def _dense_conv(self, patches, grid_idx, h, w, total):
        """Reference ``2d_conv`` branch with the sparse layer's weights: scatter, conv2d, gather."""
        B, n, C = patches.shape
        ks = self.kernel_size
        full = patches.new_zeros(B, total, C)
        full.scatter_(1, grid_idx.unsqueeze(-1).expand(-1, -1, C), patches)
        img = full.view(B * (total // (h * w)), h, w, C).permute(0, 3, 1, 2)
        wt = self.sparse_conv.weight.to(patches.dtype)
        w_conv = wt.permute(2, 1, 0).reshape(wt.shape[2], wt.shape[1], ks, ks)
        bias = self.sparse_conv.bias.to(patches.dtype) if self.sparse_conv.bias is not None else None
        out = F.conv2d(img, w_conv, bias, padding=ks // 2).permute(0, 2, 3, 1).reshape(B, total, -1)
        return torch.gather(out, 1, grid_idx.unsqueeze(-1).expand(-1, -1, out.shape[-1]))

    def forward(self, x, grid_idx, table, h, w, total, conv_impl):
        z = self.act(self.down_proj(x))
        n_special = x.shape[1] - grid_idx.shape[1]
        special, patches = z[:, :n_special], z[:, n_special:]
        if conv_impl == "svtad":
            conv = self.sparse_conv(patches.contiguous(), table, local_indices=False)
        else:
            conv = self._dense_conv(patches, grid_idx, h, w, total)
        z = torch.cat([special, conv.to(z.dtype)], dim=1)
        return self.up_proj(z) * self.gamma + x


class Block(nn.Module):
    def __init__(self, dim, num_heads, mlp_ratio, hidden, keep_rate, kernel_size):
        super().__init__()
        self.norm1 = nn.LayerNorm(dim, eps=1e-6)
        self.attn = KTPAttention(dim, num_heads, keep_rate)
        self.norm2 = nn.LayerNorm(dim, eps=1e-6)
        self.mlp = nn.Sequential(nn.Linear(dim, int(dim * mlp_ratio)), nn.GELU(), nn.Linear(int(dim * mlp_ratio), dim))
        self.adapter = SparseAdapter(dim, hidden, kernel_size)
        self.keep_rate = keep_rate

    def forward(self, x, grid_idx, table, h, w, total, conv_impl, table_impl):
        attn_out, scores = self.attn(self.norm1(x))
        x = x + attn_out
        if scores is not None:
            C = x.shape[-1]
            k_keep = min(num_keep_tokens(self.keep_rate, scores.shape[1]), scores.shape[1])
            new_table = None
            if table_impl != "svtad":
                idx = torch.topk(scores, k_keep, dim=1, largest=True)[1].sort(dim=1)[0]
            elif table is not None:
                idx, new_table = select_and_update(scores, table, k_keep)    # one kernel for the whole round
            else:
                idx = select_topk(scores, k_keep)
            kept = torch.gather(x[:, 1:], 1, idx.unsqueeze(-1).expand(-1, -1, C))
            x = torch.cat([x[:, :1], kept], dim=1)
            grid_idx = torch.gather(grid_idx, 1, idx)
            if new_table is not None:
                table = new_table
            elif table is not None:
                table = _torch_remap(table, idx)
        x = x + self.mlp(self.norm2(x))
        x = self.adapter(x, grid_idx, table, h, w, total, conv_impl)
        return x, grid_idx, table


def _torch_remap(table, idx):
    """The gather + remap of the reference block in tensor ops (:916-977), for checking the CUDA remap."""
    B, n_prev, kk = table.shape
    n_new = idx.shape[1]
    kept = torch.gather(table, 1, idx.unsqueeze(-1).expand(-1, -1, kk))
    mapping = torch.full((B * n_prev,), -1, dtype=torch.int32, device=table.device)
    off_old = (torch.arange(B, device=table.device) * n_prev).view(B, 1)
    off_new = (torch.arange(B, device=table.device) * n_new).view(B, 1)
    new_ids = (torch.arange(n_new, device=table.device).view(1, -1) + off_new).to(torch.int32)
    mapping[(idx + off_old).reshape(-1)] = new_ids.reshape(-1)
    flat = kept.reshape(-1)
    out = torch.where(flat != -1, mapping[flat.clamp(min=0).long()], torch.full_like(flat, -1))
    return out.view(B, n_new, kk)


class SparseAdapterViT(nn.Module):
    """ViT backbone with sparse adapters; defaults are the ViT-B / 160-frame shape of the benchmark configs."""

    def __init__(self, img_size=224, patch_size=16, tubelet_size=2, num_frames=160, embed_dims=768, depth=12,
                 num_heads=12, mlp_ratio=4.0, adapter_dims=192, keep_rates=None, kernel_size=3,
                 conv_impl="svtad", table_impl="svtad"):
        super().__init__()
        self.patch_size, self.tubelet_size, self.num_frames = patch_size, tubelet_size, num_frames
        self.embed_dims = embed_dims
        self.conv_impl, self.table_impl = conv_impl, table_impl
        self.kernel_size = kernel_size
        if keep_rates is None:   # one selection after the third block
            keep_rates = [1.0] * depth
            if depth > 3:
                keep_rates[3] = 0.3
        assert len(keep_rates) == depth
        self.patch_embed = nn.Conv3d(3, embed_dims, kernel_size=(tubelet_size, patch_size, patch_size),
                                     stride=(tubelet_size, patch_size, patch_size))
        grid = img_size // patch_size
        n_pos = (num_frames // tubelet_size) * grid * grid
        self.register_buffer("pos_embed", sinusoid_table(n_pos, embed_dims), persistent=False)
        self.cls_token = nn.Parameter(torch.zeros(1, 1, embed_dims))
        self.blocks = nn.ModuleList(Block(embed_dims, num_heads, mlp_ratio, adapter_dims, kr, kernel_size)
                                    for kr in keep_rates)
        self.norm = nn.LayerNorm(embed_dims, eps=1e-6)

    def forward(self, video):
        """video ``[B, 3, frames, H, W]`` -> ``[B, C, T_out + 1]`` (CLS, then per-slice mean of the kept tokens)."""
        B = video.shape[0]
        x = self.patch_embed(video)                       # [B, C, T, h, w]
        _, C, T, h, w = x.shape
        x = x.flatten(2).transpose(1, 2)                  # [B, T*h*w, C], slice-major like the reference
        total = T * h * w
        x = x + self.pos_embed[:, :total].to(x.dtype)
        x = torch.cat([self.cls_token.expand(B, -1, -1).to(x.dtype), x], dim=1)
        grid_idx = torch.arange(total, device=x.device).unsqueeze(0).repeat(B, 1)
        table = None
        if self.conv_impl == "svtad":
            table = get_initial_neighbor_indices(h, w, T, x.device, B, self.kernel_size)
        for blk in self.blocks:
            x, grid_idx, table = blk(x, grid_idx, table, h, w, total, self.conv_impl, self.table_impl)
        x = self.norm(x)
        tokens = x[:, 1:]
        frame = grid_idx // (h * w)
        summed = tokens.new_zeros(B, T, C).scatter_add_(1, frame.unsqueeze(-1).expand(-1, -1, C), tokens)
        count = tokens.new_zeros(B, T, 1).scatter_add_(1, frame.unsqueeze(-1), torch.ones_like(frame, dtype=tokens.dtype).unsqueeze(-1))
        pooled = (summed / (count + 1e-6)).permute(0, 2, 1)
        return torch.cat([x[:, :1].permute(0, 2, 1), pooled], dim=2)
