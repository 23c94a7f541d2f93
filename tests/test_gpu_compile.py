"""torch.compile around LinearStrassen, as the reference wraps its layers and models
(main_profiling.py:130-144, modded_nanogpt/data_dist_train_gpt2.py:721). The product is a
torch.library custom op, so dynamo traces the layer as one graph (fullgraph=True would raise on a
graph break) and AOT autograd builds the backward from the op's registered formula. The child process
runs with dynamo enabled; the rest of the suite keeps it disabled for the oracle's sake."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import sys, torch
sys.path.insert(0, %r)
from model.layers import LinearStrassen
import torch._dynamo
torch.manual_seed(0)
layer = LinearStrassen(512, 768, bias=True, dtype=torch.bfloat16, depth=1, device="cuda")
x0 = torch.randn(4, 256, 512, device="cuda", dtype=torch.bfloat16)
def run(mod):
    x = x0.clone().requires_grad_(True)
    mod.zero_grad(set_to_none=True)
    y = mod(x)
    y.float().square().mean().backward()
    return y.detach(), x.grad.detach(), mod.weight.grad.detach().clone(), mod.bias.grad.detach().clone()
eager = run(layer)
compiled = torch.compile(layer, fullgraph=True, backend="aot_eager")
got = run(compiled)
got2 = run(compiled)                      # second call: no recompilation, same numbers
for a, b, c in zip(eager, got, got2):
    assert torch.equal(a, b) and torch.equal(a, c)
ref = x0.double() @ layer.weight.detach().double().t() + layer.bias.detach().double()
err = ((got[0].double() - ref).norm() / ref.norm()).item()
assert err < 1.5e-2, err
explain = torch._dynamo.explain(layer)(x0)
assert explain.graph_break_count == 0, explain
assert any("b200s" in str(n.target) for g in explain.graphs for n in g.graph.nodes), "the product is not in the graph"
print("compiled ok", err)
""" % ROOT


def test_linear_strassen_under_torch_compile(built_library):
    if not torch.cuda.is_available():
        pytest.fail("this test needs a CUDA device")
    env = {k: v for k, v in os.environ.items() if k != "TORCHDYNAMO_DISABLE"}
    out = subprocess.run([sys.executable, "-c", CHILD], cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    assert "compiled ok" in out.stdout
