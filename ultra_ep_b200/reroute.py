"""Autograd bridge of the dense reroute: forward expands [T,L] probabilities to [T,P],
backward gathers the gradient of the chosen replica back to [T,L]."""

import torch


class _DenseRerouteFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, probs, routing_map, manager_runtime, layer_id):
        expanded_probs, expanded_map = manager_runtime.dense_reroute_forward(layer_id, probs, routing_map)
        ctx.mark_non_differentiable(expanded_map)
        ctx.runtime = manager_runtime
        ctx.layer_id = layer_id
        ctx.routing_map = routing_map
        ctx.expanded_map = expanded_map
        return expanded_probs, expanded_map

    @staticmethod
    def backward(ctx, grad_expanded_probs, _grad_map):
        grad = ctx.runtime.dense_reroute_backward(ctx.layer_id, grad_expanded_probs, ctx.routing_map, ctx.expanded_map)
        return grad, None, None, None
