"""Consistency chain of the EK-FAC artefacts that `bergson ekfac` writes (CPU, tiny model):
factors -> eigendecompositions -> Kronecker eigenvalues -> corrected eigenvalues."""

import pytest
import torch

from bergson_b200.__main__ import main
from bergson_b200.hessians.preconditioner import _load_full

MODEL = "native:llama-tiny?vocab_size=256"
TRAIN = "synthetic:zipf?n=24&len=16&vocab=256&seed=0&min_len=6"
QUERY = "synthetic:zipf?n=4&len=16&vocab=256&seed=1&min_len=8"


@pytest.fixture(scope="module")
def factors(tmp_path_factory):
    root = tmp_path_factory.mktemp("ekfac_chain")
    main([str(a) for a in ("ekfac", root / "run", "--model", MODEL, "--index_cfg.data.dataset", TRAIN,
                           "--hessian_pipeline_cfg.query.dataset", QUERY, "--method", "kfac",
                           "--hessian_cfg.ev_correction", "true", "--use_dataset_labels", "--token_batch_size", "64",
                           "--nproc_per_node", "1")])
    path = root / "run" / "hessian" / "kfac"
    names = ("activation_sharded", "gradient_sharded", "eigen_activation_sharded", "eigen_gradient_sharded",
             "factor_eig_a", "factor_eig_g", "eigenvalue_sharded", "eigenvalue_correction_sharded")
    out = {n: _load_full(path, n, "cpu") for n in names}
    out["total"] = float(torch.load(path / "total_processed.pt"))
    return out


def test_factors_are_symmetric_psd(factors):
    for kind in ("activation_sharded", "gradient_sharded"):
        for name, m in factors[kind].items():
            assert torch.allclose(m, m.T, atol=1e-5 * m.abs().max()), (kind, name)
            assert torch.linalg.eigvalsh(m.double()).min() > -1e-5 * m.abs().max(), (kind, name)


@pytest.mark.parametrize("side", ["a", "g"])
def test_eigendecompositions_recompose_their_factor(factors, side):
    fac = factors["activation_sharded" if side == "a" else "gradient_sharded"]
    vec = factors["eigen_activation_sharded" if side == "a" else "eigen_gradient_sharded"]
    val = factors[f"factor_eig_{side}"]
    for name, m in fac.items():
        q, lam = vec[name].double(), val[name].double()
        eye = torch.eye(q.shape[0], dtype=torch.float64)
        assert (q.T @ q - eye).abs().max() < 1e-4, name  # orthonormal columns
        # Stored eigenvalues are those of factor / T, times sqrt(T) (so that the outer product of
        # both sides carries one factor T): Q diag(lam) Q^T = factor / sqrt(T).
        recomposed = q @ torch.diag(lam) @ q.T * factors["total"] ** 0.5
        assert (recomposed - m.double()).norm() <= 1e-4 * m.double().norm() + 1e-8, name


def test_kronecker_eigenvalues_and_their_correction(factors):
    for name, kron in factors["eigenvalue_sharded"].items():
        lam_a, lam_g = factors["factor_eig_a"][name].double(), factors["factor_eig_g"][name].double()
        want = torch.outer(lam_g, lam_a)
        assert (kron.double() - want).abs().max() <= 1e-5 * want.abs().max() + 1e-10, name
        # trace identity: the Kronecker spectrum sums to tr(G) tr(A)
        tr = (factors["gradient_sharded"][name].double().trace() * factors["activation_sharded"][name].double().trace()
              / factors["total"])
        assert abs(float(kron.double().sum() - tr)) <= 1e-4 * abs(float(tr)) + 1e-10, name
        corrected = factors["eigenvalue_correction_sharded"][name]
        assert corrected.shape == kron.shape and bool((corrected >= 0).all()), name  # mean of squares
        assert float(corrected.sum()) > 0, name
