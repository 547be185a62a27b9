"""End-to-end training step of the synthetic harness on one GPU: dense warm-up step with the mean
attention maps, pattern discovery, then sparse steps -- through the reference-layout modules and
through the native block-tile modules, which must agree."""
import numpy as np
import pytest
import torch

from oracle import pattern as opat
from spion_b200 import synthetic

pytestmark = pytest.mark.gpu


def _cfg(task, batch, L, native, dtype):
    from spion_b200 import harness
    cfg = harness.task_config(task, batch, native=native, dtype=dtype)
    cfg.update(max_seq_len=L, dropout_prob=0.0, attention_dropout=0.0, threshold=0.85)
    return cfg


def _run(task, native, dtype, L=256, batch=4, steps=2, **overrides):
    from spion_b200 import harness
    cfg = _cfg(task, batch, L, native, dtype)
    cfg.update(overrides)
    tr = harness.Trainer(cfg, lr=1e-3, seed=3)
    dual = cfg["dual"]
    ids = synthetic.token_ids(5, batch, L).cuda()
    ids = (ids, synthetic.token_ids(6, batch, L).cuda()) if dual else ids
    lab = synthetic.labels(5, batch, cfg["num_classes"]).cuda()
    loss0, maps = tr.step(ids, lab, is_attn=True)                    # dense warm-up step
    assert len(maps) == cfg["num_layers"] and maps[0].shape == (L, L)
    rows = maps[0].sum(-1)
    assert torch.allclose(rows, torch.ones_like(rows), atol=1e-3)     # mean of row-stochastic maps
    mat_lst = tr.discover(maps)
    nb = L // cfg["block_size"]
    assert mat_lst.shape == (4, cfg["num_layers"], nb, nb)
    for l in range(cfg["num_layers"]):                                # same mask as the oracle on the same map
        o, _, _ = opat.discover_block_mask(maps[l].cpu().numpy(), cfg["block_size"], cfg["threshold"])
        assert np.array_equal(mat_lst[0][l].cpu().numpy(), o.astype(np.float32))
    losses = [float(loss0)]
    for _ in range(steps):
        loss, _ = tr.step(ids, lab)
        losses.append(float(loss))
    assert all(np.isfinite(losses))
    return losses, mat_lst.cpu()


def test_image_shape_fp32_reference_layout_vs_native():
    a, ma = _run("image", native=False, dtype="fp32")
    b, mb = _run("image", native=True, dtype="fp32")
    assert torch.equal(ma, mb)
    np.testing.assert_allclose(a, b, rtol=2e-4, atol=2e-4)
    assert a[-1] < a[1] + 1e-3            # training on one batch: the sparse steps do not diverge


def test_text_shape_bf16_native_with_key_padding():
    a, _ = _run("text", native=True, dtype="bf16", L=512, batch=2)
    b, _ = _run("text", native=True, dtype="fp32", L=512, batch=2)
    np.testing.assert_allclose(a, b, rtol=5e-2, atol=5e-2)


def test_retrieval_dual_tower_bf16():
    """Sparse steps with both towers as one batch of 2 B (the default of the native path) against one encoder
    call per tower (what the reference does, models/model_LRA.py): same masks, same losses to bf16 rounding."""
    a, m = _run("retrieval", native=True, dtype="bf16", L=512, batch=2)
    assert m.shape[1] == 2
    b, mb = _run("retrieval", native=True, dtype="bf16", L=512, batch=2, batch_towers=False)
    assert torch.equal(m, mb)
    np.testing.assert_allclose(a, b, rtol=3e-2, atol=3e-2)


def test_fused_layernorm_agrees_with_the_framework_operator():
    a, m = _run("text", native=True, dtype="fp32", L=256, batch=2)
    b, mb = _run("text", native=True, dtype="fp32", L=256, batch=2, fused_layernorm=False)
    assert torch.equal(m, mb)
    np.testing.assert_allclose(a, b, rtol=2e-4, atol=2e-4)


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_residual_additions_inside_the_normalisation(dtype):
    """Sparse steps with each residual addition done by the normalisation kernel that follows it (the default of
    the native path) against separate additions: same masks, same losses (fp32: the same arithmetic per element)."""
    a, m = _run("text", native=True, dtype=dtype, L=256, batch=2)
    b, mb = _run("text", native=True, dtype=dtype, L=256, batch=2, fused_add_norm=False)
    assert torch.equal(m, mb)
    tol = 2e-5 if dtype == "fp32" else 3e-2
    np.testing.assert_allclose(a, b, rtol=tol, atol=tol)


def test_bf16_parameter_copies_refreshed_once_per_step():
    """The linear layers read bf16 copies of their parameters that the trainer refreshes after every optimizer step
    (default of the native mixed-precision path); casting on every forward instead gives the same values."""
    a, m = _run("text", native=True, dtype="bf16", L=256, batch=2, steps=3)
    b, mb = _run("text", native=True, dtype="bf16", L=256, batch=2, steps=3, shadow_weights=False)
    assert torch.equal(m, mb)
    np.testing.assert_allclose(a, b, rtol=1e-6, atol=1e-6)
