import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN


def load_golden(name):
    import torch
    return torch.load(os.path.join(GOLDEN, name), map_location="cpu", weights_only=True)


def assert_close(got, ref, max_rel=2e-2, mean_abs=2e-3, what=""):
    """The path's stated tolerance against an fp32 reference on the same bf16-rounded inputs:
    max|y - ref| / max|ref| <= 2e-2 and mean|y - ref| <= 2e-3.

    Asserted as written whenever rms(ref) <= 1.  For an output whose values are larger than
    unit scale (rms > 1: GEMM outputs of N(0, 1) activations, the q / k / v projections before
    their norm, ...) the rounding of the bf16 result alone is about rms * 2^-9 per element, so an
    absolute 2e-3 cannot hold for any bf16 output; there the mean bound is taken relative to
    the output scale (2e-3 * rms).  The figures are printed either way."""
    import torch
    from oracle import complexity_oracle as oracle
    got, ref = got.float().cpu(), ref.float().cpu()
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert torch.isfinite(got).all()
    mr, ma = oracle.error_metrics(got, ref)
    rms = float(ref.double().pow(2).mean().sqrt())
    bound = mean_abs * max(1.0, rms)
    print(f"[parity] {what} max_rel={mr:.3e} mean_abs={ma:.3e} rms(ref)={rms:.3f} "
          f"mean bound={bound:.3e}{' (scaled by rms > 1)' if rms > 1.0 else ' (as written)'}")
    assert mr <= max_rel and ma <= bound, (mr, ma, rms)
    return mr, ma, rms


def build_wide_shared_layer(H, E, I_e, I_s, V, zipf_s, seed=0, device="cuda"):
    """A TokenRoutedMLP whose shared expert is wider than one routed expert (the
    expert-parallel scale-out configuration: the constructor cannot express I_s != I_e, so the
    three shared Linears are replaced — forward only calls them,
    complexity_deep/core/token_routed_mlp.py:157-160), all nine matrices N(0, 0.02) in bf16,
    bin-packed Zipf table.  Returns (module on `device`, fp32 state for the oracle, table)."""
    import torch
    import torch.nn as nn
    import complexity_deep_b200 as cd
    from oracle import complexity_oracle as oracle
    g = torch.Generator().manual_seed(seed)
    table = torch.from_numpy(oracle.build_token_mapping(
        V, E, oracle.zipf_probabilities(V, zipf_s).float()))
    with torch.device(device):
        mlp = cd.TokenRoutedMLP(H, I_e * E, E, V, True, None)
        if I_s != I_e:
            mlp.shared_gate = nn.Linear(H, I_s, bias=False)
            mlp.shared_up = nn.Linear(H, I_s, bias=False)
            mlp.shared_down = nn.Linear(I_s, H, bias=False)
    mlp = mlp.to(torch.bfloat16).eval()
    sd = {}
    with torch.no_grad():
        for name, prm in mlp.named_parameters():
            w = (torch.randn(prm.shape, generator=g) * 0.02).to(torch.bfloat16)
            prm.copy_(w)
            sd[name] = w.float()
        mlp.token_to_expert.copy_(table)
    sd["token_to_expert"] = table
    return mlp, sd, table
