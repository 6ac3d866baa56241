"""The row-wise and attention kernels that Falalix brought, each against plain PyTorch float32."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rnd(*shape, seed=0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g).to(dtype).to(DEV)


@pytest.mark.parametrize("act", ["none", "silu", "relu2", "sigmoid", "tanh", "softplus"])
@pytest.mark.parametrize("in_dt,out_dt", [(torch.float32, torch.float32), (torch.float32, torch.bfloat16),
                                          (torch.bfloat16, torch.bfloat16)])
def test_rows_act(act, in_dt, out_dt):
    from rllm_b200.csrc import ops
    wide = rnd(37, 50, seed=1, dtype=in_dt) * 3
    a = wide[:, 7:40]                                   # a column slice: rows 50 apart
    bias, mul = rnd(33, seed=2), rnd(37, 33, seed=3)
    out = torch.full((37, 40), 7.0, dtype=out_dt, device=DEV)
    ops.rows_act(a, out[:, 2:35], act=act, bias=bias, mul=mul, mul_act="sigmoid")
    z = a.float() + bias
    f = {"none": lambda z: z, "silu": lambda z: z * torch.sigmoid(z), "relu2": lambda z: torch.relu(z) ** 2,
         "sigmoid": torch.sigmoid, "tanh": torch.tanh, "softplus": torch.nn.functional.softplus}[act]
    want = f(z) * torch.sigmoid(mul)
    tol = 1e-6 if out_dt == torch.float32 else 8e-3
    assert torch.allclose(out[:, 2:35].float(), want, rtol=tol, atol=tol)
    assert float(out[:, :2].float().min()) == 7.0 and float(out[:, 35:].float().max()) == 7.0     # nothing beside the slice


def test_axpby_cat2_and_scaled_norm():
    from rllm_b200.csrc import ops
    x, y = rnd(19, 44, seed=4), rnd(19, 44, seed=5)
    out = torch.empty_like(x)
    ops.axpby(0.6, x, -1.7, y, out)
    assert torch.allclose(out, 0.6 * x - 1.7 * y, rtol=1e-6, atol=1e-6)
    delta = rnd(19, 44, seed=6, dtype=torch.bfloat16)
    both = torch.empty((19, 88), dtype=torch.bfloat16, device=DEV)
    ops.cat2_cast(x, y, both, delta=delta, delta_scale=0.3)
    want = torch.cat([x + 0.3 * delta.float(), y], 1)
    assert torch.allclose(both.float(), want, rtol=8e-3, atol=8e-3)
    w = 1 + 0.1 * rnd(44, seed=7)
    xs, normed = x.clone(), torch.empty((19, 44), dtype=torch.float32, device=DEV)
    ops.add_rms_norm(xs, y, w, normed, 1e-5, delta_scale=0.25)
    v = x + 0.25 * y
    assert torch.allclose(xs, v, rtol=1e-6, atol=1e-6)                                  # the stream got the scaled sum
    assert torch.allclose(normed, v / torch.sqrt((v * v).mean(-1, keepdim=True) + 1e-5) * w, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n", [5, 200])                  # few tokens: 1,024 threads a row; many: 256
def test_qkv_rownorm_store(dtype, n):
    """Bias, RMS norm over the whole q row and the whole k row, queries out, keys and values (heads of
    another size) into pages; the projection has more columns behind v that are left alone."""
    from rllm_b200.csrc import ops
    H, G, dk, dv, bs, pages, eps = 3, 2, 24, 40, 8, 40, 1e-5
    wq, wk, wv = H * dk, G * dk, G * dv
    wide = rnd(n, wq + wk + wv + 13, seed=8)
    bias = rnd(wq + wk + wv, seed=9)
    qn, kn = 1 + 0.2 * rnd(wq, seed=10), 1 + 0.2 * rnd(wk, seed=11)
    slots = torch.randperm(pages * bs, generator=torch.Generator().manual_seed(1))[:n].to(torch.int32).to(DEV)
    slots[1] = -1                                        # a padding row writes nothing
    q = torch.empty((n, wq), dtype=dtype, device=DEV)
    kc = torch.zeros((pages, G, bs, dk), dtype=dtype, device=DEV)
    vc = torch.zeros((pages, G, bs, dv), dtype=dtype, device=DEV)
    ops.qkv_rownorm_store(wide[:, :wq + wk + wv], bias, qn, kn, slots, q, kc, vc, H, G, dk, dv, bs, eps)
    z = wide[:, :wq + wk + wv] + bias
    unit = lambda r: r / torch.sqrt((r * r).mean(-1, keepdim=True) + eps)
    tol = 2e-6 if dtype == torch.float32 else 8e-3
    assert torch.allclose(q.float(), unit(z[:, :wq]) * qn, rtol=tol, atol=tol)
    kw, vw = (unit(z[:, wq:wq + wk]) * kn).view(n, G, dk), z[:, wq + wk:].reshape(n, G, dv)
    for t in range(n):
        s = int(slots[t])
        if s < 0:
            continue
        assert torch.allclose(kc[s // bs, :, s % bs].float(), kw[t], rtol=tol, atol=tol)
        assert torch.allclose(vc[s // bs, :, s % bs].float(), vw[t], rtol=tol, atol=tol)
    written = set(int(s) for s in slots if s >= 0)
    assert int((kc.float().abs().sum((1, 3)) > 0).sum()) == len(written)                 # no other place was touched


@pytest.mark.parametrize("window,keep", [(0, 0), (9, 0), (9, 4), (9, 40), (70, 3)])
def test_plain_attention_with_kept_keys_and_value_heads_of_their_own(window, keep):
    from rllm_b200.csrc import ops
    H, G, dk, dv, bs, T = 4, 2, 24, 56, 8, 150
    q = rnd(T, H * dk, seed=12)
    k, v = rnd(T, G, dk, seed=13), rnd(T, G, dv, seed=14)
    pages = -(-T // bs)
    order = torch.randperm(pages, generator=torch.Generator().manual_seed(2))
    kc = torch.zeros((pages, G, bs, dk), device=DEV)
    vc = torch.zeros((pages, G, bs, dv), device=DEV)
    for p in range(T):
        kc[order[p // bs], :, p % bs] = k[p]
        vc[order[p // bs], :, p % bs] = v[p]
    out = torch.empty((T, H * dv), device=DEV)
    pos = torch.arange(T, dtype=torch.int32, device=DEV)
    ops.paged_attention_generic(q, kc, vc, out, pos, torch.zeros(T, dtype=torch.int32, device=DEV),
                                order.to(torch.int32).to(DEV).view(1, -1), H, G, dk, bs, 0.3, window, keep, dv)
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    see = (j <= i) & ((i - j < window) | (j < keep) if window else torch.ones(T, T, dtype=torch.bool))
    want = torch.empty(T, H, dv, device=DEV)
    for h in range(H):
        s = (q.view(T, H, dk)[:, h] @ k[:, h // (H // G)].T) * 0.3
        s = s.masked_fill(~see.to(DEV), -math.inf)
        want[:, h] = torch.softmax(s, -1) @ v[:, h // (H // G)]
    assert torch.allclose(out, want.view(T, H * dv), rtol=2e-5, atol=2e-5)
