"""Library-only grid sample (sort + searchsorted instead of the table, plain
torch indexing), usable on any device: the cross-check the reference also ships
(flex_gemm/ops/grid_sample/grid_sample_torch.py:8-154; there the table lookups
still run its CUDA kernels)."""
import torch


def _lookup(coords: torch.Tensor, shape, pts: torch.Tensor) -> torch.Tensor:
    """Row of each integer point (b, x, y, z) [M, 4] or -1."""
    C, W, H, D = [int(s) for s in shape[-4:]]
    c = coords.to(torch.int64)
    key = ((c[:, 0] * W + c[:, 1]) * H + c[:, 2]) * D + c[:, 3]
    skey, order = torch.sort(key)
    p = pts.to(torch.int64)
    ok = (p[:, 1] >= 0) & (p[:, 1] < W) & (p[:, 2] >= 0) & (p[:, 2] < H) & (p[:, 3] >= 0) & (p[:, 3] < D)
    pkey = ((p[:, 0] * W + p[:, 1]) * H + p[:, 2]) * D + p[:, 3]
    if skey.numel() == 0:
        return torch.full_like(pkey, -1)
    pos = torch.searchsorted(skey, pkey).clamp_(0, skey.numel() - 1)
    ok &= skey[pos] == pkey
    return torch.where(ok, order[pos], torch.full_like(pos, -1))


def grid_sample_3d_torch(feats: torch.Tensor, coords: torch.Tensor, shape: torch.Size, grid: torch.Tensor, mode: str = "trilinear") -> torch.Tensor:
    assert mode in ["nearest", "trilinear"], "Invalid interpolation mode"
    B, L = grid.shape[:2]
    C = feats.shape[1]
    q = grid.float()
    b = torch.arange(B, device=grid.device).view(B, 1, 1).expand(B, L, 1)
    if mode == "nearest":
        pts = torch.cat([b, q.to(torch.int32).to(torch.int64)], dim=2).view(-1, 4)   # truncation towards zero, as the kernels do
        idx = _lookup(coords, shape, pts)
        out = torch.where((idx >= 0).unsqueeze(1), feats[idx.clamp_min(0)], torch.zeros((), dtype=feats.dtype, device=feats.device))
        return out.view(B, L, C)
    base = torch.floor(q - 0.5)
    acc = torch.zeros((B * L, C), dtype=torch.float32, device=feats.device)
    wsum = torch.zeros(B * L, dtype=torch.float32, device=feats.device)
    for k in range(8):
        off = torch.tensor([k & 1, (k >> 1) & 1, (k >> 2) & 1], dtype=torch.float32, device=grid.device)
        corner = base + off
        pts = torch.cat([b, corner.to(torch.int64)], dim=2).view(-1, 4)
        idx = _lookup(coords, shape, pts)
        w = torch.prod(1 - torch.abs(q - corner - 0.5), dim=-1).view(-1)
        w = torch.where(idx >= 0, w, torch.zeros_like(w))
        acc += w.unsqueeze(1) * feats[idx.clamp_min(0)].float()
        wsum += w
    return (acc / wsum.clamp_min(1e-12).unsqueeze(1)).to(feats.dtype).view(B, L, C)
