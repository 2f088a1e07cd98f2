"""CPU-only API checks against outputs of the unmodified reference (tests/golden/api.npz):
LSQActivation is plain torch and runs where the tensors live (coset/core/layers.py:117-137)."""
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN


@pytest.mark.parametrize("tag,bits_,alpha", [("a", 8, 1.3), ("b", 4, 0.7)])
def test_lsq_activation_matches_reference(tag, bits_, alpha):
    from coset_b200.core.layers import LSQActivation, ste_clip, ste_round
    g = np.load(os.path.join(GOLDEN, "api.npz"))
    act = LSQActivation(bits_, alpha)
    assert act.qmax == 2 ** (bits_ - 1) - 1
    x = torch.from_numpy(g[f"lsq_{tag}_x"]).requires_grad_(True)
    y = act(x)
    (y * torch.from_numpy(g[f"lsq_{tag}_t"])).sum().backward()
    assert np.array_equal(y.detach().numpy(), g[f"lsq_{tag}_y"])
    assert np.array_equal(x.grad.numpy(), g[f"lsq_{tag}_dx"])
    assert np.allclose(act.alpha.grad.numpy(), g[f"lsq_{tag}_dalpha"], rtol=1e-6)
    # straight-through helpers: forward value of the op, identity gradient
    z = torch.tensor([0.4, 1.6, -2.5], requires_grad=True)
    r = ste_round(z)
    r.sum().backward()
    assert torch.equal(r.detach(), torch.round(z.detach())) and torch.equal(z.grad, torch.ones(3))
    z.grad = None
    c = ste_clip(z, -1.0, 1.0)
    c.sum().backward()
    assert torch.equal(c.detach(), z.detach().clamp(-1, 1)) and torch.equal(z.grad, torch.ones(3))
