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


def rotation_boundary_probes(hgroup, exponents=(-9, 0, 6), steps=8):
    """fp32 rows of 128 whose rotation is known exactly, for driving the quantiser's rounding boundaries
    THROUGH the Hadamard butterfly.  Each row holds one 32-element scale group with two non-zero rotated
    values: a maximum that fixes the group's scale so that the top code is reachable, and a probe placed on a
    grid of `2*steps+1` neighbouring values around the preimage of one E2M1 rounding boundary
    (0.25 ... 5.0, both signs).  The row is x = H t / g with t that sparse vector; every butterfly partial sum
    of such an x is a small multiple of the two values, so the fp32 butterfly returns t bit for bit (the
    function checks this).  The probe grid is one ulp of the probe when rotation and scale group do not
    overlap (hgroup 16: maximum and probe sit in different rotation groups), else the coarsest spacing that
    keeps maximum +- probe exact in fp32.  Returns (x [rows, 128] fp32, t [rows, 128] fp32)."""
    import numpy as np

    g = hgroup
    c = np.float32(1.0 / np.sqrt(g))
    H = np.ones((1, 1))
    while H.shape[0] < g:
        H = np.block([[H, H], [H, -H]])
    rows_x, rows_t = [], []
    i = 0
    for q in exponents:
        # rotated maximum y = t_max * c in (5s, 6s]: 1.9 * 2^q with s = (4/3) 2^(q-2) gives 5.7 s
        t_max = np.float32(np.round(1.9 * 2.0 ** q / float(c) * 2.0 ** (6 - q)) * 2.0 ** (q - 6))
        e = int(np.floor(np.log2(float(np.float32(t_max * c)))))
        s = np.float32(2.0 ** (e - 2)) / np.float32(0.75)
        for b in (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0):
            ideal = b * float(s) / float(c)
            if g == 16:
                grid = float(np.spacing(np.float32(ideal)))
            else:
                grid = float(np.spacing(t_max)) * 2.0
            centre = np.round(ideal / grid) * grid
            for j in range(-steps, steps + 1):
                for sign in (1.0, -1.0):
                    tk = np.float32(sign * (centre + j * grid))
                    sg = i % 4
                    p0 = (7 * i) % (16 if g == 16 else 32)
                    p1 = 16 + (5 * i) % 16 if g == 16 else (p0 + 1 + i % 31) % 32
                    t = np.zeros(128, dtype=np.float64)
                    t[sg * 32 + p0] = float(t_max) * (1.0 if i % 3 else -1.0)
                    t[sg * 32 + p1] = float(tk)
                    x = (t.reshape(-1, g) @ H) / g
                    rows_x.append(x.reshape(-1))
                    rows_t.append(t)
                    i += 1
    x64 = np.stack(rows_x)
    x32 = x64.astype(np.float32)
    assert np.array_equal(x32.astype(np.float64), x64), "probe rows are not exact in fp32"
    return torch.from_numpy(x32), torch.from_numpy(np.stack(rows_t).astype(np.float32))
