"""The oracle's optimizer step against the reference's own known answers and invariants
(optimizer/optim_test.go, optimizer/sinkhorn_test.go)."""
import numpy as np


def test_adamw_exact_value(oracle):
    # optim_test.go:10-27: param 1, grad 1, lr 0.01 -> 0.99
    p = np.array([1.0], np.float32); m = np.zeros(1, np.float32); v = np.zeros(1, np.float32)
    oracle.adamw_step(p, np.array([1.0], np.float32), m, v, 1, 0.01, 0.9, 0.999, 1e-8)
    assert abs(p[0] - 0.99) <= 1e-5


def test_adamw_reduces_quadratic_loss(oracle):
    # optim_test.go:29-49
    p = np.ones(100, np.float32); m = np.zeros(100, np.float32); v = np.zeros(100, np.float32)
    before = float(np.sum(p.astype(np.float64) ** 2))
    for step in range(1, 11):
        oracle.adamw_step(p, 2 * p, m, v, step, 0.05, 0.9, 0.999, 1e-8)
    assert float(np.sum(p.astype(np.float64) ** 2)) < before


def test_sinkhorn_single_row_normalization(oracle):
    # sinkhorn_test.go:12-25: K=1, unit row [0.6, 0.8] times sqrt(columns)
    p = np.zeros(2, np.float32); mom = np.zeros(2, np.float32)
    oracle.sinkhorn_step(p, np.array([3, 4], np.float32), mom, 1, 2, lr=1, momentum=0, gamma=1, steps=1, tau=0, eps=1e-20)
    assert np.allclose(p, [-np.sqrt(2) * 0.6, -np.sqrt(2) * 0.8], atol=1e-5)


def test_sinkhorn_masks_near_zero_rows(oracle):
    # sinkhorn_test.go:29-44
    p = np.zeros(4, np.float32); mom = np.zeros(4, np.float32)
    oracle.sinkhorn_step(p, np.array([3, 4, 0, 0], np.float32), mom, 2, 2, lr=1, momentum=0, gamma=1, steps=1, tau=0.5, eps=1e-20)
    assert p[2] == 0 and p[3] == 0 and p[0] != 0 and p[1] != 0


def test_sinkhorn_rows_have_unit_rms(oracle):
    # sinkhorn_test.go:48-68
    p = np.zeros(12, np.float32); mom = np.zeros(12, np.float32)
    g = np.array([1e-3, 2e-3, 3e-3, 4, 5, 6, 7, 8, 9, 0.1, 0.2, 0.3], np.float32)
    oracle.sinkhorn_step(p, g, mom, 4, 3, lr=1, momentum=0, gamma=1, steps=11, tau=0, eps=1e-20)
    rms = np.sqrt(np.mean(p.reshape(4, 3).astype(np.float64) ** 2, axis=1))
    assert np.all(np.abs(rms - 1) <= 1e-3)


def test_muon_tall_and_wide(oracle):
    # optim_test.go:66-119: finite, every element moves, second moment positive; per-column state for a wide matrix
    rng = np.random.default_rng(1)
    for rows, cols in ((6, 3), (3, 8)):
        p = (rng.standard_normal(rows * cols) * 0.1).astype(np.float32); g = (rng.standard_normal(rows * cols) * 0.1).astype(np.float32)
        before = p.copy(); mom = np.zeros_like(p); sec = np.zeros(max(rows, cols), np.float32)
        oracle.muon_step(p, g, mom, sec, rows, cols, lr=0.01)
        assert np.all(np.isfinite(p)) and np.all(p != before)
        assert np.all(sec > 0) and np.all(np.isfinite(sec))


def test_muon_update_is_orthogonalised(oracle):
    """Polar Express drives the singular values of the update toward one: with lr 1, no decay and zero parameters the
    step is -U with U^T U close to a multiple of the identity (optimizer/muon.go:57-86)."""
    rng = np.random.default_rng(2)
    rows, cols = 24, 8
    g = rng.standard_normal(rows * cols).astype(np.float32)
    p = np.zeros(rows * cols, np.float32); mom = np.zeros_like(p); sec = np.zeros(rows, np.float32)
    oracle.muon_step(p, g, mom, sec, rows, cols, lr=1.0, momentum=0.0)
    sv = np.linalg.svd(p.reshape(rows, cols).astype(np.float64), compute_uv=False)
    assert sv.max() / sv.min() < 2.0      # raw gradient: condition number ~3-4


def test_model_optimizer_routing_and_zero_grad(oracle):
    from gonano_b200 import synthetic
    cfg = synthetic.dense_config("tiny")
    m = oracle.Model(**cfg)
    rng = np.random.default_rng(3)
    for name, value in synthetic.fill_weights(m.names, m.shape, 1, std=0.1):
        m.param(name)[:] = value
        m.grad(name)[:] = (rng.standard_normal(value.size) * 0.01).astype(np.float32)
    before = {n: m.param(n).copy() for n in m.names}
    opt = oracle.Optimizer(m)
    opt.step()
    for n in m.names:
        assert np.all(np.isfinite(m.param(n))) and np.any(m.param(n) != before[n]), n
        assert not np.any(m.grad(n))
    # Sinkhorn applies no weight decay and moves every unmasked row by gamma * lr * (unit-RMS row): lm_head lr = 0.004 * 0.05 * (d/768)^-0.5
    d = (m.param("lm_head.weight") - before["lm_head.weight"]).reshape(m.shape("lm_head.weight")).astype(np.float64)
    rms = np.sqrt(np.mean(d ** 2, axis=1))
    dim_scale = (cfg["embed_dim"] / 768.0) ** -0.5      # model/optimizer.go:108
    assert np.allclose(rms[rms > 0], 0.18 * 0.004 * 0.05 * dim_scale, rtol=2e-2)
