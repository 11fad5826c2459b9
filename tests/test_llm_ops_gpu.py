"""Bandwidth kernels of the Llama step against fp32 PyTorch restatements."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _close(got, ref, rtol=2e-2, atol=2e-2):
    err = (got.float() - ref.float()).abs().max().item()
    assert err <= rtol * ref.float().abs().max().item() + atol, err


@pytest.mark.parametrize("T,H", [(64, 256), (33, 4096), (16, 2048), (8, 8192)])
@pytest.mark.parametrize("with_res", [False, True])
def test_rmsnorm_fwd_bwd(T, H, with_res):
    from aws_ofi_nccl_b200.ops import llm

    x = torch.randn(T, H, device="cuda").bfloat16().requires_grad_(True)
    r = torch.randn(T, H, device="cuda").bfloat16().requires_grad_(True) if with_res else None
    w = (1 + 0.1 * torch.randn(H, device="cuda")).bfloat16().requires_grad_(True)
    y, h = llm.rmsnorm(x, w, 1e-5, residual=r)
    dy = torch.randn_like(y)
    dh = torch.randn_like(y)
    (y * dy).sum().backward(retain_graph=False) if not with_res else ((y * dy).sum() + (h * dh).sum()).backward()
    xf = x.detach().float().requires_grad_(True)
    rf = r.detach().float().requires_grad_(True) if with_res else None
    wf = w.detach().float().requires_grad_(True)
    hf = xf + rf if with_res else xf
    hq = hf + (hf.bfloat16().float() - hf).detach() if with_res else hf  # kernel normalises the rounded sum
    yf = hq * torch.rsqrt(hq.pow(2).mean(-1, keepdim=True) + 1e-5) * wf
    loss = (yf * dy.float()).sum() + ((hf * dh.float()).sum() if with_res else 0)
    loss.backward()
    _close(y, yf)
    _close(x.grad, xf.grad, atol=5e-2)
    _close(w.grad, wf.grad, atol=0.3)
    if with_res:
        _close(h, hf)
        _close(r.grad, rf.grad, atol=5e-2)


def test_swiglu():
    from aws_ofi_nccl_b200.ops import llm

    gu = torch.randn(96, 2 * 512, device="cuda").bfloat16().requires_grad_(True)
    out = llm.swiglu(gu)
    d = torch.randn_like(out)
    out.backward(d)
    g = gu.detach().float().requires_grad_(True)
    ref = F.silu(g[:, :512]) * g[:, 512:]
    ref.backward(d.float())
    _close(out, ref)
    _close(gu.grad, g.grad)


def test_cross_entropy_and_grad():
    from aws_ofi_nccl_b200.ops import llm

    T, V = 48, 128256 // 8 + 8
    logits = (torch.randn(T, V, device="cuda") * 2).bfloat16()
    tgt = torch.randint(0, V, (T,), device="cuda")
    lf = logits.float().requires_grad_(True)
    ref = F.cross_entropy(lf, tgt)
    ref.backward()
    lg = logits.clone().requires_grad_(True)
    l2 = lg * 1.0
    loss = llm.cross_entropy(l2, tgt)
    loss.backward()
    assert abs(loss.item() - ref.item()) < 2e-3
    assert (lg.grad.float() - lf.grad).abs().max().item() < 2e-4


def test_embedding_fwd_bwd():
    from aws_ofi_nccl_b200.ops import llm

    table = torch.randn(100, 64, device="cuda").bfloat16().requires_grad_(True)
    ids = torch.randint(0, 100, (4, 16), device="cuda")
    out = llm.embedding(ids, table)
    assert torch.equal(out, table.detach()[ids])
    d = torch.randn_like(out)
    out.backward(d)
    ref = torch.zeros(100, 64, device="cuda").index_add_(0, ids.reshape(-1), d.reshape(-1, 64).float())
    _close(table.grad, ref, atol=6e-2)


def test_rope_roundtrip_and_reference():
    from aws_ofi_nccl_b200.ops import llm

    T, nh, hd, seq = 64, 6, 128, 32
    x = torch.randn(T, nh, hd, device="cuda").bfloat16()
    inv = 1.0 / (10000 ** (torch.arange(0, hd, 2, device="cuda").float() / hd))
    ang = torch.outer(torch.arange(seq, device="cuda").float(), inv)
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    y = llm.rope_(x.clone(), cos, sin, seq)
    pos = torch.arange(T, device="cuda") % seq
    c, s = cos[pos].view(T, 1, hd // 2), sin[pos].view(T, 1, hd // 2)
    a, b = x.float()[..., : hd // 2], x.float()[..., hd // 2:]
    ref = torch.cat([a * c - b * s, b * c + a * s], -1)
    _close(y, ref)
    xr = x.clone().requires_grad_(True)
    z = llm.rope_(xr * 1.0, cos, sin, seq)
    d = torch.randn_like(z)
    z.backward(d)
    dr = d.float()
    da, db = dr[..., : hd // 2], dr[..., hd // 2:]
    gref = torch.cat([da * c + db * s, db * c - da * s], -1)
    _close(xr.grad, gref)


def test_adamw_matches_torch():
    from aws_ofi_nccl_b200.ops import llm

    n = 8 * 1000
    p = torch.randn(n, device="cuda").bfloat16()
    g = torch.randn(n, device="cuda").bfloat16()
    master = p.float()
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    pr = torch.nn.Parameter(master.clone())
    opt = torch.optim.AdamW([pr], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for step in range(1, 4):
        pr.grad = g.float()
        opt.step()
        gg = g.clone()
        llm.adamw_step(p, gg, m, v, master, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step)
        assert gg.abs().max().item() == 0  # zero_grad fused
    assert torch.allclose(master, pr.detach(), rtol=1e-4, atol=1e-5)
    assert torch.allclose(p.float(), pr.detach(), rtol=1e-2, atol=1e-2)
