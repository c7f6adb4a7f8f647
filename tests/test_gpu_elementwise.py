"""Numerics of the HBM-bound kernels against plain PyTorch fp32 references."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda", 0)


@pytest.mark.parametrize("gdtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n", [1, 7, 4096, 100003])
def test_fused_sgd_matches_torch(gdtype, n):
    from tips_b200.ops.optim import FusedSGD
    torch.manual_seed(0)
    p_ref = torch.randn(n, device=_dev())
    p = torch.nn.Parameter(p_ref.clone().to(gdtype))
    ref = torch.nn.Parameter(p.detach().float().clone())
    opt = FusedSGD([p], lr=0.1, momentum=0.9, weight_decay=1e-2, nesterov=True)
    ropt = torch.optim.SGD([ref], lr=0.1, momentum=0.9, weight_decay=1e-2, nesterov=True)
    for _ in range(3):
        g = torch.randn(n, device=_dev()).to(gdtype)
        p.grad = g.clone()
        ref.grad = g.float()
        opt.step()
        ropt.step()
    master = opt._flat[0].master[:n]
    assert torch.allclose(master, ref.detach(), atol=1e-5, rtol=1e-5)
    tol = 1e-5 if gdtype == torch.float32 else 2e-2
    assert torch.allclose(p.detach().float(), ref.detach(), atol=tol, rtol=tol)


@pytest.mark.parametrize("n", [5, 1024, 33333])
def test_fused_adamw_matches_torch(n):
    from tips_b200.ops.optim import FusedAdamW
    torch.manual_seed(1)
    p = torch.nn.Parameter(torch.randn(n, device=_dev()))
    ref = torch.nn.Parameter(p.detach().clone())
    opt = FusedAdamW([p], lr=1e-2, weight_decay=0.05)
    ropt = torch.optim.AdamW([ref], lr=1e-2, weight_decay=0.05)
    for _ in range(4):
        g = torch.randn(n, device=_dev())
        p.grad = g.clone()
        ref.grad = g.clone()
        opt.step()
        ropt.step()
    assert torch.allclose(p.detach(), ref.detach(), atol=2e-5, rtol=1e-4)


def test_pack_unpack_roundtrip():
    from tips_b200.parallel.buckets import build_buckets
    torch.manual_seed(2)
    params = [torch.nn.Parameter(torch.randn(s, device=_dev())) for s in [(3, 5), (17,), (64, 33), (1,)]]
    for p in params:
        p.grad = torch.randn_like(p)
    buckets = build_buckets(params, threshold_bytes=1 << 20, wire_dtype="bf16")
    assert len(buckets) == 1
    b = buckets[0]
    b.pack(scale=0.5)
    for i, p in enumerate(b.params):
        assert torch.allclose(b.view_of(i).float(), (p.grad * 0.5).to(torch.bfloat16).float())
    b.pack(scale=0.5, accumulate=True)
    for i, p in enumerate(b.params):
        assert torch.allclose(b.view_of(i).float(), p.grad, atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape", [(8, 64, 14, 14), (4, 24, 7, 5), (2, 256, 9, 9)])
@pytest.mark.parametrize("relu,res", [(False, False), (True, False), (True, True)])
def test_batchnorm_fwd_bwd(dtype, shape, relu, res):
    from tips_b200.ops.norm import BatchNorm2d
    torch.manual_seed(3)
    dev = _dev()
    bn = BatchNorm2d(shape[1], relu=relu).to(dev)
    with torch.no_grad():
        bn.weight.uniform_(0.5, 1.5)
        bn.bias.uniform_(-0.5, 0.5)
    x = torch.randn(shape, device=dev).to(dtype).contiguous(memory_format=torch.channels_last).requires_grad_()
    r = torch.randn(shape, device=dev).to(dtype).contiguous(memory_format=torch.channels_last).requires_grad_() if res else None
    y = bn(x, residual=r)
    dy = torch.randn_like(y)
    y.backward(dy)
    # fp32 reference
    xr = x.detach().float().requires_grad_()
    rr = r.detach().float().requires_grad_() if res else None
    w = bn.weight.detach().clone().requires_grad_()
    b = bn.bias.detach().clone().requires_grad_()
    yr = torch.nn.functional.batch_norm(xr, None, None, w, b, True, 0.1, bn.eps)
    if res:
        yr = yr + rr
    if relu:
        yr = torch.relu(yr)
    yr.backward(dy.float())
    tol = 2e-4 if dtype == torch.float32 else 6e-2
    assert torch.allclose(y.float(), yr, atol=tol, rtol=tol)
    assert torch.allclose(x.grad.float(), xr.grad, atol=tol, rtol=tol)
    gtol = 1e-3 if dtype == torch.float32 else 0.25
    assert torch.allclose(bn.weight.grad, w.grad, atol=gtol, rtol=5e-2)
    assert torch.allclose(bn.bias.grad, b.grad, atol=gtol, rtol=5e-2)
    if res:
        assert torch.allclose(r.grad.float(), rr.grad, atol=tol, rtol=tol)
    m = x.numel() // shape[1]
    xm = x.detach().float().transpose(0, 1).reshape(shape[1], -1)
    assert torch.allclose(bn.running_mean, 0.1 * xm.mean(1), atol=1e-3)
    assert torch.allclose(bn.running_var, 0.9 + 0.1 * xm.var(1, unbiased=True), atol=1e-2)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rows,cols", [(3, 64), (257, 1024), (64, 768), (20000, 1024), (5000, 256)])
def test_layernorm_fwd_bwd(dtype, rows, cols):
    from tips_b200.ops.norm import LayerNorm
    torch.manual_seed(4)
    dev = _dev()
    ln = LayerNorm(cols).to(dev)
    with torch.no_grad():
        ln.weight.uniform_(0.5, 1.5)
        ln.bias.uniform_(-0.5, 0.5)
    x = torch.randn(rows, cols, device=dev).to(dtype).requires_grad_()
    y = ln(x)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr = x.detach().float().requires_grad_()
    w = ln.weight.detach().clone().requires_grad_()
    b = ln.bias.detach().clone().requires_grad_()
    yr = torch.nn.functional.layer_norm(xr, (cols,), w, b, ln.eps)
    yr.backward(dy.float())
    tol = 2e-4 if dtype == torch.float32 else 6e-2
    assert torch.allclose(y.float(), yr, atol=tol, rtol=tol)
    assert torch.allclose(x.grad.float(), xr.grad, atol=tol, rtol=tol)
    assert torch.allclose(ln.weight.grad, w.grad, atol=0.3 if dtype != torch.float32 else 1e-3, rtol=5e-2)
    assert torch.allclose(ln.bias.grad, b.grad, atol=0.3 if dtype != torch.float32 else 1e-3, rtol=5e-2)


@pytest.mark.parametrize("act", ["relu", "gelu", None])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_bias_act(act, dtype):
    from tips_b200.ops.pointwise import bias_act
    torch.manual_seed(5)
    dev = _dev()
    x = torch.randn(37, 256, device=dev).to(dtype).requires_grad_()
    bias = torch.randn(256, device=dev).to(dtype).requires_grad_()
    y = bias_act(x, bias, act)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr = x.detach().float().requires_grad_()
    br = bias.detach().float().requires_grad_()
    z = xr + br
    yr = torch.relu(z) if act == "relu" else torch.nn.functional.gelu(z) if act == "gelu" else z
    yr.backward(dy.float())
    tol = 1e-4 if dtype == torch.float32 else 5e-2
    assert torch.allclose(y.float(), yr, atol=tol, rtol=tol)
    assert torch.allclose(x.grad.float(), xr.grad, atol=tol, rtol=tol)
    assert torch.allclose(bias.grad.float(), br.grad, atol=0.3 if dtype != torch.float32 else 1e-3, rtol=5e-2)


def test_losses():
    from tips_b200.ops.pointwise import sigmoid_bce_loss, softmax_cross_entropy
    torch.manual_seed(6)
    dev = _dev()
    z = torch.randn(1000, device=dev).requires_grad_()
    t = (torch.rand(1000, device=dev) < 0.25).float()
    loss = sigmoid_bce_loss(z, t)
    loss.backward()
    zr = z.detach().clone().requires_grad_()
    lr = torch.nn.functional.binary_cross_entropy_with_logits(zr, t)
    lr.backward()
    assert torch.allclose(loss, lr, atol=1e-5)
    assert torch.allclose(z.grad, zr.grad, atol=1e-6)
    logits = torch.randn(33, 1000, device=dev).to(torch.bfloat16).requires_grad_()
    labels = torch.randint(0, 1000, (33,), device=dev)
    labels[5] = -100
    loss = softmax_cross_entropy(logits, labels)
    loss.backward()
    lg = logits.detach().float().requires_grad_()
    ref = torch.nn.functional.cross_entropy(lg, labels, ignore_index=-100)
    ref.backward()
    assert torch.allclose(loss, ref, atol=2e-3)
    assert torch.allclose(logits.grad.float(), lg.grad, atol=2e-3)


@pytest.mark.parametrize("dtype,rows,k", [(torch.bfloat16, 8192, 256), (torch.bfloat16, 777, 520),
                                          (torch.float32, 1000, 36)])
def test_one_unit_output_layer_fused_with_bce(dtype, rows, k):
    """linear1_sigmoid_bce_loss against torch in fp32: loss, dx, dw, db; the input is a column slice of a wider
    matrix (a row pitch larger than k) and the upstream gradient is not 1."""
    from tips_b200.ops.pointwise import linear1_sigmoid_bce_loss
    torch.manual_seed(rows)
    dev = _dev()
    wide = torch.randn(rows, k + 8, device=dev).to(dtype)
    x = wide[:, :k].detach().requires_grad_()
    w = (torch.randn(1, k, device=dev) * 0.1).to(dtype).requires_grad_()
    b = torch.randn(1, device=dev).to(dtype).requires_grad_()
    t = (torch.rand(rows, device=dev) < 0.25).float()
    loss = linear1_sigmoid_bce_loss(x, w, b, t)
    (loss * 3.0).backward()
    xr, wr, br = (v.detach().float().requires_grad_() for v in (x, w, b))
    ref = torch.nn.functional.binary_cross_entropy_with_logits(torch.nn.functional.linear(xr, wr, br).view(-1), t)
    (ref * 3.0).backward()
    low = dtype != torch.float32
    assert torch.allclose(loss, ref, atol=1e-4 if low else 1e-5, rtol=1e-4)
    assert torch.allclose(x.grad.float(), xr.grad, atol=1e-6 if not low else 2e-6, rtol=1e-2 if low else 1e-4)
    assert torch.allclose(w.grad.float(), wr.grad, atol=2e-3 if low else 1e-5, rtol=1e-2 if low else 1e-4)
    assert torch.allclose(b.grad.float(), br.grad, atol=2e-3 if low else 1e-5, rtol=1e-2 if low else 1e-4)


@pytest.mark.parametrize("n,c,h,w", [(2, 64, 16, 16), (3, 8, 7, 9), (1, 16, 1, 5), (4, 64, 112, 112)])
def test_maxpool_3x3_s2(n, c, h, w):
    from tips_b200.ops.pool import max_pool_3x3_s2
    torch.manual_seed(n * 100 + h)
    dev = torch.device("cuda", 0)
    x = torch.randn(n, c, h, w, device=dev).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    x.requires_grad_()
    y = max_pool_3x3_s2(x)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr = x.detach().float().requires_grad_()
    yr = torch.nn.functional.max_pool2d(xr, 3, stride=2, padding=1)
    yr.backward(dy.float())
    assert torch.equal(y.float(), yr)
    # ties between equal bf16 values may pick different positions; the gradient mass per window is the same
    # (each bf16 gradient carries its own rounding error, so the tolerance grows with the image area)
    assert torch.allclose(x.grad.float().sum(dim=(2, 3)), xr.grad.sum(dim=(2, 3)), rtol=2e-2, atol=2e-2 + 1e-4 * h * w)
    mismatch = (x.grad.float() - xr.grad).abs() > 1e-2
    assert mismatch.float().mean() < 0.02


@pytest.mark.parametrize("b,s,heads,d", [(2, 128, 4, 64), (3, 77, 2, 32)])
def test_packed_attention_matches_plain_sdpa(b, s, heads, d):
    from tips_b200.ops.attention import packed_attention
    torch.manual_seed(b * s)
    dev = torch.device("cuda", 0)
    h = heads * d
    qkv = torch.randn(b, s, 3 * h, device=dev).to(torch.bfloat16).requires_grad_()
    dy = torch.randn(b, s, h, device=dev).to(torch.bfloat16)
    y = packed_attention(qkv, heads)
    y.backward(dy)
    ref_in = qkv.detach().float().requires_grad_()
    q, k, v = ref_in.view(b, s, 3, heads, d).permute(2, 0, 3, 1, 4)
    yr = torch.nn.functional.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(b, s, h)
    yr.backward(dy.float())
    assert torch.allclose(y.float(), yr, atol=3e-2, rtol=3e-2)
    assert torch.allclose(qkv.grad.float(), ref_in.grad, atol=5e-2, rtol=5e-2)


def test_copy4d_permutes():
    from tips_b200.ops.attention import copy4d
    dev = torch.device("cuda", 0)
    src = torch.randn(3, 5, 7, 64, device=dev).to(torch.bfloat16)
    dst = torch.empty(3, 7, 5, 64, device=dev, dtype=torch.bfloat16)
    copy4d(src.transpose(1, 2), dst)
    assert torch.equal(dst, src.transpose(1, 2).contiguous())
    packed = torch.zeros(3, 7, 3, 5, 64, device=dev, dtype=torch.bfloat16)
    copy4d(src.transpose(1, 2), packed[:, :, 1])
    assert torch.equal(packed[:, :, 1], src.transpose(1, 2)) and float(packed[:, :, 0].abs().sum()) == 0.0


def test_bert_layer_matches_plain_pytorch():
    """One encoder layer (packed attention, residual adds fused into the layer norms, gradients of the block inputs
    summed inside the GEMMs) against the same computation written with plain PyTorch ops in fp32."""
    import torch.nn.functional as F
    from tips_b200.models.bert import BertLayer
    torch.manual_seed(11)
    dev = torch.device("cuda", 0)
    hidden, heads, ffn, b, s = 256, 4, 1024, 4, 128
    layer = BertLayer(hidden, heads, ffn).to(dev).to(torch.bfloat16)
    x = (torch.randn(b, s, hidden, device=dev) * 0.5).to(torch.bfloat16).requires_grad_()
    dy = torch.randn(b, s, hidden, device=dev).to(torch.bfloat16)
    y = layer(x)
    y.backward(dy)
    p = {k: v.detach().float() for k, v in layer.named_parameters()}
    xr = x.detach().float().requires_grad_()
    qkv = F.linear(xr, p["qkv.weight"], p["qkv.bias"]).view(b, s, 3, heads, hidden // heads).permute(2, 0, 3, 1, 4)
    att = F.scaled_dot_product_attention(qkv[0], qkv[1], qkv[2]).transpose(1, 2).reshape(b, s, hidden)
    h1 = F.layer_norm(xr + F.linear(att, p["proj.weight"], p["proj.bias"]), (hidden,), p["ln1.weight"], p["ln1.bias"], 1e-12)
    f = F.linear(F.gelu(F.linear(h1, p["fc1.weight"], p["fc1.bias"])), p["fc2.weight"], p["fc2.bias"])
    yr = F.layer_norm(h1 + f, (hidden,), p["ln2.weight"], p["ln2.bias"], 1e-12)
    yr.backward(dy.float())
    assert torch.allclose(y.float(), yr, atol=6e-2, rtol=6e-2)
    ga, gb = x.grad.float(), xr.grad
    assert float((ga * gb).sum() / (ga.norm() * gb.norm())) > 0.995
    assert (ga - gb).abs().max() <= 0.1 * max(1.0, float(gb.abs().max()))


def test_make_subgraph_replays_our_kernels():
    """A function made of this package's kernels, captured once and replayed on new inputs."""
    from tips_b200.ops import norm
    from tips_b200.utils.misc import executing_eagerly, make_subgraph
    dev = torch.device("cuda", 0)
    ln = norm.LayerNorm(1024).to(dev).to(torch.bfloat16)
    seen = []

    def fn(x):
        seen.append(executing_eagerly())
        with torch.no_grad():
            return ln(x) * 2

    x0 = torch.randn(512, 1024, device=dev).to(torch.bfloat16)
    g = make_subgraph(fn, x0)
    assert seen[-1] is False and seen[0] is True  # warm-up ran eagerly, the last call was the capture
    for seed in (1, 2):
        torch.manual_seed(seed)
        x = torch.randn(512, 1024, device=dev).to(torch.bfloat16)
        out = g(x).clone()
        with torch.no_grad():
            ref = ln(x) * 2
        assert torch.equal(out, ref)
    assert g.replays == 2


@pytest.mark.parametrize("dtype,shape", [(torch.bfloat16, (5, 2048, 7, 7)), (torch.float32, (3, 12, 4, 9))])
def test_global_average_pool(dtype, shape):
    from tips_b200.ops.pool import global_avg_pool
    torch.manual_seed(1)
    dev = _dev()
    x = torch.randn(shape, device=dev).to(dtype).contiguous(memory_format=torch.channels_last).requires_grad_()
    y = global_avg_pool(x)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr = x.detach().float().requires_grad_()
    yr = xr.mean(dim=(2, 3))
    yr.backward(dy.float())
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert y.shape == yr.shape and torch.allclose(y.float(), yr, atol=tol, rtol=tol)
    assert torch.allclose(x.grad.float(), xr.grad, atol=tol, rtol=tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_sum(dtype):
    """embed_sum against torch indexing in fp32: values, and the gradients of the token table (duplicate ids),
    the position table (longer than the sequence) and the type row."""
    from tips_b200.ops.pointwise import embed_sum
    torch.manual_seed(2)
    dev = _dev()
    vocab, seq, hidden, batch = 300, 24, 64, 5
    tok = torch.randn(vocab, hidden, device=dev).to(dtype).requires_grad_()
    pos = torch.randn(seq + 8, hidden, device=dev).to(dtype).requires_grad_()
    typ = torch.randn(2, hidden, device=dev).to(dtype).requires_grad_()
    ids = torch.randint(0, 40, (batch, seq), device=dev)          # many duplicates
    x = embed_sum(ids, tok, pos, typ[0])
    dx = torch.randn_like(x)
    x.backward(dx)
    tr, pr, yr = (t.detach().float().requires_grad_() for t in (tok, pos, typ))
    xr = tr[ids] + pr[:seq][None] + yr[0]
    xr.backward(dx.float())
    tol = 1e-5 if dtype == torch.float32 else 6e-2
    assert torch.allclose(x.float(), xr, atol=tol, rtol=tol)
    assert torch.allclose(tok.grad.float(), tr.grad, atol=tol * 4, rtol=tol)
    assert torch.allclose(pos.grad.float(), pr.grad, atol=tol, rtol=tol)
    assert torch.allclose(typ.grad.float(), yr.grad, atol=tol * 8, rtol=tol)
