"""The layer-level CPU oracle against the reference's own BitLinear forward/backward."""
import numpy as np
import torch

from oracle import metis_layer as ML


def test_layer_oracle_matches_reference_forward_and_backward(layer_golden):
    g = {k: torch.from_numpy(np.asarray(v)) for k, v in layer_golden.items() if k != "rank"}
    y, saved = ML.forward(g["x"], g["U"], g["S"], g["V"], g["R"], g["bias"])
    torch.testing.assert_close(y, g["y"], rtol=1e-5, atol=1e-5)
    grads = ML.backward(g["grad_out"], saved, g["U"], g["S"], has_bias=True)
    for name in ("dx", "dR", "dV", "dU", "ds", "dbias"):
        torch.testing.assert_close(grads[name], g[name], rtol=2e-5, atol=2e-5, msg=name)


def test_split_reconstructs_the_weight(layer_golden):
    W = torch.from_numpy(layer_golden["W"])
    U, S, V, R = ML.split_weight(W, int(layer_golden["rank"]))
    torch.testing.assert_close(U @ torch.diag(S) @ V + R, W, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(R, torch.from_numpy(layer_golden["R"]), rtol=1e-4, atol=1e-6)
