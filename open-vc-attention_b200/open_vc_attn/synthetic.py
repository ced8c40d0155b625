"""Seeded synthetic inputs with the shapes and value structure of the published benchmark.

The reference measures on private BF16 captures of a video-diffusion denoising step
(docs/performance.md:15 of the reference); only their shapes are public.  These generators stand in
for them: same S, H, D and dtype, and the value structure the captures are described to have.
"""

import torch


def video_dit_qkv(length, heads, *, seed, dtype=torch.bfloat16, device="cuda", first_head=0):
    """Q,K ~ N(0,1) with 4 of 128 channels per head scaled x8 (outlier channels) and each token scaled by
    LogNormal(0, 0.3); V ~ N(mu_h, 1) with a per-head channel mean mu_h ~ N(0, sigma=2).

    Every head is drawn from its own generator seeded with ``seed + first_head + h``, so a rank that
    holds heads [h0, h1) of a larger tensor generates exactly those heads' values.
    """
    q = torch.empty(length, heads, 128, dtype=dtype, device=device)
    k = torch.empty_like(q)
    v = torch.empty_like(q)
    for h in range(heads):
        g = torch.Generator(device=device).manual_seed(seed + first_head + h)
        for dst in (q, k):
            x = torch.randn(length, 128, generator=g, device=device)
            idx = torch.randperm(128, generator=g, device=device)[:4]
            x[:, idx] *= 8
            x *= torch.exp(0.3 * torch.randn(length, 1, generator=g, device=device))
            dst[:, h] = x.to(dtype)
        mu = 2.0 * torch.randn(1, 128, generator=g, device=device)
        v[:, h] = (torch.randn(length, 128, generator=g, device=device) + mu).to(dtype)
    return q, k, v


def student_t_values(length, heads, *, seed, dof=3.0, dtype=torch.bfloat16, device="cuda"):
    """V ~ Student-t(dof) (heavy tails stress FP8 rounding; the V-repair configuration)."""
    g = torch.Generator(device=device).manual_seed(seed)
    normal = torch.randn(length, heads, 128, generator=g, device=device)
    chi2 = torch.zeros_like(normal)
    for _ in range(int(dof)):
        chi2 += torch.randn(length, heads, 128, generator=g, device=device).pow(2)
    return (normal / torch.sqrt(chi2 / dof)).to(dtype)
