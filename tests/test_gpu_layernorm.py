"""The library's layer normalisation (csrc/layernorm.cu) against torch.nn.functional.layer_norm in fp32
(the operator the reference's encoder uses: models/model_transformer.py): outputs, input gradients and the
weight / bias gradients, fp32 and bf16 outputs, every supported width, row counts that do not divide the grid."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("N", [64, 128, 256, 512])
@pytest.mark.parametrize("M", [1, 37, 4096, 70001])
def test_forward_backward_fp32(M, N):
    from spion_b200.layernorm import FusedLayerNorm
    g = torch.Generator().manual_seed(M + N)
    x = (torch.randn(M, N, generator=g) * 3 + 0.5).cuda().requires_grad_(True)
    dy = torch.randn(M, N, generator=g).cuda()
    mod = FusedLayerNorm(N).cuda()
    with torch.no_grad():
        mod.weight.copy_(torch.randn(N, generator=g)); mod.bias.copy_(torch.randn(N, generator=g))
    y = mod(x)
    y.backward(dy)
    xr = x.detach().clone().requires_grad_(True)
    w = mod.weight.detach().clone().requires_grad_(True); b = mod.bias.detach().clone().requires_grad_(True)
    yr = torch.nn.functional.layer_norm(xr, (N,), w, b, 1e-5)
    yr.backward(dy)
    assert float((y.detach() - yr.detach()).abs().max()) <= 2e-5
    assert float((x.grad - xr.grad).abs().max()) <= 2e-5 * max(1.0, float(xr.grad.abs().max()))
    # sums over M rows: tolerance relative to the magnitude of the sum
    assert float((mod.weight.grad - w.grad).abs().max()) <= 1e-4 * max(1.0, float(w.grad.abs().max()))
    assert float((mod.bias.grad - b.grad).abs().max()) <= 1e-4 * max(1.0, float(b.grad.abs().max()))


def test_bf16_output_under_autocast_and_3d_input():
    from spion_b200.layernorm import FusedLayerNorm
    B, L, N = 3, 1000, 64
    g = torch.Generator().manual_seed(5)
    x = torch.randn(B, L, N, generator=g).cuda().requires_grad_(True)
    mod = FusedLayerNorm(N, bf16_out=True).cuda()
    lin = torch.nn.Linear(N, 32).cuda()
    with torch.autocast(device_type="cuda", dtype=torch.bfloat16):
        y = mod(x)
        assert y.dtype == torch.bfloat16 and y.shape == x.shape
        out = lin(y)
    out.float().sum().backward()
    xr = x.detach().clone().requires_grad_(True)
    with torch.autocast(device_type="cuda", dtype=torch.bfloat16):
        yr = torch.nn.functional.layer_norm(xr, (N,), mod.weight.detach(), mod.bias.detach(), 1e-5)
        outr = lin(yr)
    outr.float().sum().backward()
    assert float((y.detach().float() - yr.detach().float()).abs().max()) <= 2e-2
    assert float((x.grad - xr.grad).abs().max()) <= 2e-2 * float(xr.grad.abs().max())
    assert mod(x.detach()).dtype == torch.float32           # outside autocast the output stays fp32


def test_results_do_not_depend_on_the_run():
    """The weight / bias gradients are sums in a fixed order: two runs give identical bits."""
    from spion_b200.layernorm import FusedLayerNorm
    g = torch.Generator().manual_seed(9)
    x = torch.randn(50000, 64, generator=g).cuda()
    dy = torch.randn(50000, 64, generator=g).cuda()
    grads = []
    for _ in range(2):
        mod = FusedLayerNorm(64).cuda()
        xx = x.clone().requires_grad_(True)
        mod(xx).backward(dy)
        grads.append((mod.weight.grad.clone(), mod.bias.grad.clone(), xx.grad.clone()))
    for a, b in zip(*grads):
        assert torch.equal(a, b)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("N", [64, 128, 512])
def test_linear_with_column_sum_bias_gradient(N, dtype):
    """BiasGradLinear against nn.Linear with the same parameters: output, dX, dW and the bias gradient (the only
    part that runs on the library's kernel), in fp32 and under bf16 autocast."""
    from spion_b200.layernorm import BiasGradLinear
    g = torch.Generator().manual_seed(N)
    B, L, K = 3, 1111, 64
    x = torch.randn(B, L, K, generator=g).cuda()
    dy = torch.randn(B, L, N, generator=g).cuda()
    ref = torch.nn.Linear(K, N).cuda()
    mine = BiasGradLinear(K, N).cuda()
    mine.load_state_dict(ref.state_dict())
    outs = []
    for mod in (ref, mine):
        xx = x.clone().requires_grad_(True)
        with torch.autocast(device_type="cuda", dtype=torch.bfloat16, enabled=dtype == torch.bfloat16):
            y = mod(xx)
        y.backward(dy.to(y.dtype))
        outs.append((y.detach().float(), xx.grad, mod.weight.grad, mod.bias.grad))
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    for name, a, b in zip(("y", "dx", "dW", "db"), *outs):
        scale = max(1.0, float(a.abs().max()))
        assert float((a - b).abs().max()) <= tol * scale, name


@pytest.mark.parametrize("V,N,B,L,dtype", [
    (256, 64, 16, 4096, torch.float32),      # the retrieval / text tasks' table
    (256, 64, 3, 1000, torch.float32),       # tokens not a multiple of the staged batch
    (512, 32, 1, 777, torch.float32),        # odd token count: the last id goes by a plain load
    (48, 128, 5, 301, torch.bfloat16),
    (64, 256, 2, 515, torch.float32),
])
def test_token_embedding_weight_gradient(V, N, B, L, dtype):
    """TokenEmbedding against nn.Embedding with the same table: forward bits, weight gradient against an fp64
    scatter-sum (1e-5 of the largest entry for fp32 rows), identical bits on a second run.  Half of the tokens are
    id 0 in runs, as padded sequences have them."""
    from spion_b200.layernorm import TokenEmbedding
    g = torch.Generator().manual_seed(V + N)
    ids = torch.randint(0, V, (B, L), generator=g)
    ids[:, L // 2:] = 0
    ids = ids.cuda()
    dy = torch.randn(B, L, N, generator=g).cuda().to(dtype)
    ref = torch.nn.Embedding(V, N).cuda()
    mine = TokenEmbedding(V, N).cuda()
    mine.load_state_dict(ref.state_dict())
    assert mine.served(ids)
    assert torch.equal(mine(ids), ref(ids))
    grads = []
    for _ in range(2):
        mine.weight.grad = None
        y = mine(ids)
        y.backward(dy.to(y.dtype))
        grads.append(mine.weight.grad.clone())
    assert torch.equal(grads[0], grads[1])
    want = torch.zeros(V, N, dtype=torch.float64, device="cuda")
    want.index_add_(0, ids.reshape(-1), dy.to(torch.float32).double().reshape(-1, N))
    err = float((grads[0].double() - want).abs().max())
    assert err <= 1e-5 * max(1.0, float(want.abs().max()))


def test_token_embedding_falls_back_for_large_tables():
    from spion_b200.layernorm import TokenEmbedding
    mod = TokenEmbedding(30000, 64).cuda()
    ids = torch.randint(0, 30000, (2, 128)).cuda()
    assert not mod.served(ids)
    mod(ids).sum().backward()
    assert mod.weight.grad is not None


@pytest.mark.parametrize("res_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("N", [64, 256])
def test_add_norm_matches_separate_addition_and_normalisation(N, res_dtype):
    """FusedLayerNorm.add_norm(x, res) = (x + res, norm(x + res)), forward bits and every gradient, when the sum
    also feeds a later consumer (the next residual connection) and when it does not."""
    from spion_b200.layernorm import FusedLayerNorm
    g = torch.Generator().manual_seed(N)
    M = 3333
    x0 = torch.randn(M, N, generator=g).cuda()
    r0 = torch.randn(M, N, generator=g).cuda().to(res_dtype)
    dy = torch.randn(M, N, generator=g).cuda()
    dskip = torch.randn(M, N, generator=g).cuda()
    for use_sum in (True, False):
        outs = []
        for fused in (False, True):
            mod = FusedLayerNorm(N).cuda()
            with torch.no_grad():
                mod.weight.copy_(torch.linspace(0.5, 1.5, N)); mod.bias.copy_(torch.linspace(-1, 1, N))
            x = x0.clone().requires_grad_(True)
            r = r0.clone().requires_grad_(True)
            if fused:
                s, y = mod.add_norm(x, r)
            else:
                s = r + x
                y = mod(s)
            loss = (y * dy).sum() + ((s * dskip).sum() if use_sum else 0.0)
            loss.backward()
            outs.append((s.detach(), y.detach(), x.grad, r.grad.float(), mod.weight.grad, mod.bias.grad))
        for name, a, b in zip(("sum", "y", "dx", "dres", "dweight", "dbias"), *outs):
            if name in ("sum", "y"):
                assert torch.equal(a, b), name
            else:
                scale = max(1.0, float(a.abs().max()))
                tol = 1e-5 if (name != "dres" or res_dtype == torch.float32) else 8e-3
                assert float((a - b).abs().max()) <= tol * scale, (name, use_sum)


@pytest.mark.parametrize("B,L,Lmax", [(3, 512, 512), (2, 300, 1024)])
def test_token_plus_position_embedding_in_one_kernel(B, L, Lmax):
    """TokenEmbedding.with_positions against ``tok(ids) + pos.weight[:L][None]``: same bits forward, same gradients of
    both tables (the position table may have more rows than the sequences use)."""
    from spion_b200.layernorm import TokenEmbedding
    V, N = 256, 64
    g = torch.Generator().manual_seed(L)
    ids = torch.randint(0, V, (B, L), generator=g).cuda()
    dy = torch.randn(B, L, N, generator=g).cuda()
    tok = TokenEmbedding(V, N).cuda()
    pos = torch.nn.Embedding(Lmax, N).cuda()
    outs = []
    for fused in (False, True):
        tok.weight.grad = None
        pos.weight.grad = None
        y = tok.with_positions(ids, pos.weight) if fused else torch.nn.functional.embedding(ids, tok.weight) + pos.weight[:L][None]
        y.backward(dy)
        outs.append((y.detach(), tok.weight.grad.clone(), pos.weight.grad.clone()))
    assert torch.equal(outs[0][0], outs[1][0])
    for a, b in zip(outs[0][1:], outs[1][1:]):
        assert float((a - b).abs().max()) <= 1e-5 * max(1.0, float(a.abs().max()))
