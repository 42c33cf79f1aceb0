"""Every public name of the reference's Python modules can be imported from the module of the same path here, and the
ones that compute something compute what the reference's do (checked against plain PyTorch formulas)."""
import ast
import importlib
import math
import os

import pytest
import torch

# the reference's source tree: a checkout named by B200MOE_REFERENCE_TREE (covers the side car under rl/ as well),
# else the copy installed for the benchmark's reference arm; without either the walk is skipped
_HERE = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REFERENCE = os.environ.get("B200MOE_REFERENCE_TREE") or os.path.join(_HERE, "baseline", "_ref")
NOT_CARRIED: dict = {}     # per reference file: names deliberately absent here (none)


def _reference_modules():
    if not os.path.isdir(REFERENCE):
        return []
    found = []
    for folder, dirs, files in os.walk(REFERENCE):
        dirs[:] = [d for d in dirs if not d.startswith(".") and d not in ("tests", "__pycache__", "kubernetes")
                   and not d.endswith(".dist-info")]
        for name in files:
            if name.endswith(".py"):
                found.append(os.path.relpath(os.path.join(folder, name), REFERENCE))
    return sorted(found)


@pytest.mark.parametrize("relative", _reference_modules())
def test_public_names_of_the_reference_exist_here(relative):
    with open(os.path.join(REFERENCE, relative), encoding="utf-8") as handle:
        tree = ast.parse(handle.read())
    names = [node.name for node in tree.body if isinstance(node, (ast.FunctionDef, ast.ClassDef))]
    module_name = relative[:-3].replace(os.sep, ".")
    if module_name.endswith(".__init__"):
        module_name = module_name[:-9]
    module = importlib.import_module(module_name)
    missing = [n for n in names if not hasattr(module, n) and n not in NOT_CARRIED.get(relative, ())]
    assert not missing, f"{relative}: {missing}"


def _argument_names(node):
    return [a.arg for a in node.args.args] + [a.arg for a in node.args.kwonlyargs]


def _accepts(callable_, wanted):
    """Names of ``wanted`` that ``callable_`` cannot take by keyword."""
    import inspect
    try:
        have = inspect.signature(callable_).parameters
    except (TypeError, ValueError):
        return []
    if any(p.kind in (p.VAR_KEYWORD, p.VAR_POSITIONAL) for p in have.values()):
        return []
    if getattr(callable_, "PARAMETERS", None):
        have = set(have) | set(callable_.PARAMETERS)
    return [name for name in wanted if name not in have]


@pytest.mark.parametrize("relative", _reference_modules())
def test_methods_and_argument_names_of_the_reference_exist_here(relative):
    """Every method of a reference class exists on the class here, and every function or method takes the
    reference's argument names (so calls by keyword keep working)."""
    with open(os.path.join(REFERENCE, relative), encoding="utf-8") as handle:
        tree = ast.parse(handle.read())
    module_name = relative[:-3].replace(os.sep, ".")
    module = importlib.import_module(module_name[:-9] if module_name.endswith(".__init__") else module_name)
    problems = []
    for node in tree.body:
        here = getattr(module, node.name, None) if isinstance(node, (ast.FunctionDef, ast.ClassDef)) else None
        if here is None:
            continue
        if isinstance(node, ast.FunctionDef):
            target = getattr(here, "__call__", here) if getattr(here, "PARAMETERS", None) else here
            missing = _accepts(target, _argument_names(node)) if not getattr(here, "PARAMETERS", None) else \
                [n for n in _argument_names(node) if n not in here.PARAMETERS]
            if missing:
                problems.append(f"{node.name}: no argument {missing}")
            continue
        for method in (n for n in node.body if isinstance(n, ast.FunctionDef)):
            if not hasattr(here, method.name):
                problems.append(f"{node.name}.{method.name}: missing")
                continue
            wanted = [n for n in _argument_names(method) if n not in ("self", "cls", "ctx")]
            missing = _accepts(getattr(here, method.name), wanted)
            if missing:
                problems.append(f"{node.name}.{method.name}: no argument {missing}")
    assert not problems, f"{relative}: {problems}"


def test_attention_functions_take_queries_first_and_match_the_formula():
    from implementation.kernels.attention import (FlashAttentionFunc, FlashAttentionTritonFunc, attention_forward,
                                                  attention_pytorch)
    from b200moe.models.layers import Attention_Flash
    torch.manual_seed(0)
    B, S, D = 2, 32, 16
    q, k, v = (torch.randn(B, S, D, requires_grad=True) for _ in range(3))
    for causal in (False, True):
        visible = torch.arange(S)[:, None] >= torch.arange(S)[None, :] if causal else torch.ones(S, S, dtype=torch.bool)
        scores = (q @ k.transpose(-1, -2) / math.sqrt(D)).masked_fill(~visible, float("-inf"))
        want = torch.softmax(scores, -1) @ v
        grad_out = torch.randn_like(want)
        want_grads = torch.autograd.grad(want, (q, k, v), grad_out, retain_graph=True)
        for function in (FlashAttentionFunc, FlashAttentionTritonFunc):
            got_out = function.apply(q, k, v, causal)
            assert torch.allclose(got_out, want, atol=1e-5)
            for a, b in zip(torch.autograd.grad(got_out, (q, k, v), grad_out), want_grads):
                assert torch.allclose(a, b, atol=1e-5)
        lse = torch.logsumexp(scores, -1).detach()
        got = attention_pytorch(q.detach(), k.detach(), v.detach(), want.detach(), grad_out, lse,
                                visible.float().unsqueeze(0))
        assert got[3] is None
        for a, b in zip(got[:3], want_grads):
            assert torch.allclose(a, b, atol=1e-5)
        out, row_lse = torch.empty(B, S, D), torch.empty(B, S)
        attention_forward[(2, B)](q.detach(), k.detach(), v.detach(), out, row_lse, *([0] * 14), S, S,
                                  1 / math.sqrt(D), D, 16, 16, causal)
        assert torch.allclose(out, want, atol=1e-5) and torch.allclose(row_lse, lse, atol=1e-5)
    # the layer hands (k, q, v) to a function whose first argument holds the queries, like the reference's
    layer_out = Attention_Flash()(k.detach(), q.detach(), v.detach(), None)
    assert torch.allclose(layer_out, torch.softmax(k @ q.transpose(-1, -2) / math.sqrt(D), -1) @ v, atol=1e-5)


def test_host_snapshots_of_model_and_optimizer_state():
    from implementation.train_utils import move_model_state, move_optimizer_state
    model = torch.nn.Linear(4, 3)
    optimizer = torch.optim.AdamW(model.parameters(), lr=1e-2)
    model(torch.randn(2, 4)).sum().backward()
    optimizer.step()
    weights = move_model_state(model)
    assert set(weights) == {"weight", "bias"} and all(t.device.type == "cpu" for t in weights.values())
    assert torch.equal(weights["weight"], model.weight.detach()) and weights["weight"] is not model.weight
    state = move_optimizer_state(optimizer)
    assert state["param_groups"][0]["lr"] == 1e-2 and set(state["state"]) == {0, 1}
    assert torch.equal(state["state"][0]["exp_avg"], optimizer.state_dict()["state"][0]["exp_avg"])
    model.weight.data.zero_()                      # the snapshot is a copy
    assert float(weights["weight"].abs().sum()) > 0
    fresh = torch.optim.AdamW(torch.nn.Linear(4, 3).parameters(), lr=1.0)
    fresh.load_state_dict(state)
    assert fresh.param_groups[0]["lr"] == 1e-2
