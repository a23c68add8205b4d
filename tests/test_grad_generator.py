"""Incremental gradients (grad_generator) and the C++ execution-order analysis.
Modelled on python/tests/test_grad_generator.py of the reference."""
import torch

from monarch_b200.gradient_generator import (GradGenerator, grad_function, grad_generator,
                                             gradient_execution_order)


def test_grads_match_autograd_and_order():
    torch.manual_seed(0)
    ws = [torch.randn(4, 4, requires_grad=True) for _ in range(4)]
    x = torch.randn(2, 4)
    h = x
    for w in ws:
        h = torch.tanh(h @ w)
    loss = h.sum()
    expect = torch.autograd.grad(loss, ws, retain_graph=True)
    got = list(grad_generator(loss, list(reversed(ws))))
    for g, e in zip(reversed(got), expect):
        assert torch.allclose(g, e)
    # the last layer's weight is used first in backward, so its gradient is ready first
    assert gradient_execution_order([loss], ws) == [3, 2, 1, 0]


def test_unused_inputs_yield_none_and_empty():
    a = torch.randn(3, requires_grad=True)
    b = torch.randn(3, requires_grad=True)
    out = (a * 2).sum()
    ga, gb = list(grad_generator(out, [a, b]))
    assert torch.allclose(ga, torch.full((3,), 2.0)) and gb is None
    assert list(grad_generator(out, [])) == []


def test_grad_generator_builder_and_grad_roots():
    a = torch.randn(3, requires_grad=True)
    b = torch.randn(3, requires_grad=True)
    y = a * b
    g = GradGenerator()
    g.root(y, torch.ones(3) * 2)
    g.grad({"a": a})
    g.grad([b])
    trees = list(g)
    assert torch.allclose(trees[0][0], 2 * a) and torch.allclose(trees[1]["a"], 2 * b)


def test_grad_function_continuation():
    @grad_function
    def double(x):
        y = x * 2

        def backward(gy):
            return gy * 2 + 0 * y
        return y, backward

    x = torch.randn(5, requires_grad=True)
    double(x).sum().backward()
    assert torch.allclose(x.grad, torch.full((5,), 2.0))


def test_errors_in_backward_propagate():
    class Boom(torch.autograd.Function):
        @staticmethod
        def forward(ctx, x):
            return x.clone()

        @staticmethod
        def backward(ctx, g):
            raise RuntimeError("backward exploded")

    x = torch.randn(2, requires_grad=True)
    import pytest
    with pytest.raises(RuntimeError, match="exploded"):
        list(grad_generator(Boom.apply(x).sum(), [x]))
