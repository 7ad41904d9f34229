"""Seeded synthetic inputs shared by the CPU and GPU tests (generated in fp32 on the CPU,
then cast, so both sides see identical bits)."""
import torch


def normal_weight(rows, cols, seed=0, std=0.02, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(rows, cols, generator=g) * std).to(dtype)


def outlier_activations(rows, cols, seed=1, dtype=torch.bfloat16):
    """Student-t(nu=4) * 0.5 with 1 % of the channels scaled by 20."""
    g = torch.Generator().manual_seed(seed)
    z = torch.randn(rows, cols, generator=g)
    chi = torch.randn(rows, cols, 4, generator=g).pow(2).sum(-1)
    x = z / torch.sqrt(chi / 4) * 0.5
    g2 = torch.Generator().manual_seed(seed + 1)
    idx = torch.randperm(cols, generator=g2)[: max(1, cols // 100)]
    x[:, idx] *= 20
    return x.to(dtype)


def correlated_activations(tokens, d, seed=6, dtype=torch.bfloat16):
    """X = Z A + 0.1 E with a rank-64 mixing: makes the Hessian far from diagonal."""
    g = torch.Generator().manual_seed(seed)
    z = torch.randn(tokens, 64, generator=g)
    a = torch.randn(64, d, generator=g) / 8
    e = torch.randn(tokens, d, generator=g)
    return (z @ a + 0.1 * e).to(dtype)


def edge_case_rows(cols=128):
    """Rows that exercise rounding ties, zero groups, near-power-of-two maxima, extremes.
    Intended for hadamard_group = 0 so the values reach the quantiser unchanged."""
    rows = []
    base = torch.zeros(cols)
    rows.append(base.clone())                                   # all zero
    r = base.clone(); r[::2] = -0.0; rows.append(r)             # signed zeros
    ties = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, -0.25, -0.75,
                         -1.25, -1.75, -2.5, -3.5, -5.0, -6.0, 0.0, 0.1, 7.0, -7.0, 5.5, 4.5, 2.75, 2.25, 0.3, 0.7])
    for scale in (1.0, 2.0 ** -7, 2.0 ** 5, 3.0, 0.75, 4.0 / 3.0):
        r = base.clone()
        for g0 in range(0, cols, 32):
            r[g0:g0 + 32] = ties * scale
        rows.append(r)
    # maxima a few ulps below powers of two (log2 rounding artefact of the E8M0 exponent)
    for k in (-20, -3, 0, 1, 7, 30):
        for ulps in (1, 2, 3, 8, 40, 300):
            p = torch.tensor(2.0 ** k, dtype=torch.float32)
            v = p
            for _ in range(ulps):
                v = torch.nextafter(v, torch.tensor(0.0))
            r = torch.linspace(-1, 1, cols) * float(v) * 0.9
            r[5] = float(v)
            rows.append(r.float())
    for mag in (1e-30, 1e-38, 3e-39, 1e-42, 1e30, 1e37):
        g = torch.Generator().manual_seed(int(abs(torch.tensor(mag).log10().item())))
        rows.append((torch.randn(cols, generator=g) * mag).float())
    return torch.stack(rows).float()
