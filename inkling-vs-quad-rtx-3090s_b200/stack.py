"""A stack of MoE blocks decoded one token at a time under CUDA-graph replay: the
skeleton of the reference's decode loop (my_inkling/decode_graph.py:7-58 around
my_inkling/model.py:672-675) with everything but the MoE block reduced to the residual
add and RMS norm between blocks."""
from __future__ import annotations

import torch
from torch import nn

from .kernels import StackDescriptor, add_rmsnorm
from .layer import FusedMoE, ResidentExperts
from .synthetic import make_expert_banks, make_layer_params


class MoEStack(nn.Module):
    def __init__(self, layers: list[FusedMoE], hidden: int, eps: float = 1e-6):
        super().__init__()
        self.layers = nn.ModuleList(layers)
        self.hidden, self.eps = hidden, eps
        dev = layers[0].router_weight.device
        self.norm_weight = torch.ones(hidden, dtype=torch.bfloat16, device=dev)
        self._tokens = 0
        self._fused = None
        # one launch for the whole stack, on one GPU or across tensor-parallel ranks
        self.one_launch = all(layer.one_launch_supported() for layer in layers)

    @classmethod
    def synthetic(cls, n_layers: int, hidden: int, intermediate: int, experts: int, n_shared: int, top_k: int,
                  device, seed: int = 0, device_mesh=None, rank: int = 0, world: int = 1,
                  route_scale: float = 8.0, bias_std: float = 0.0):
        layers = []
        for layer in range(n_layers):
            banks = make_expert_banks(experts, hidden, intermediate, device, seed + 1000 * layer, rank=rank, world=world)
            p = make_layer_params(hidden, intermediate, experts, n_shared, device, seed + 1000 * layer, rank=rank,
                                  world=world, bias_std=bias_std)
            ex = ResidentExperts(hidden, intermediate // world, device_mesh, banks.weights)
            ex.banks = banks
            layers.append(FusedMoE(p["router_weight"], p["router_bias"], p["global_scale"], route_scale, top_k,
                                   p["shared_gate"], p["shared_up"], p["shared_down"], ex, device_mesh))
        return cls(layers, hidden)

    def _reserve(self, tokens: int) -> None:
        if tokens > self._tokens:
            dev = self.norm_weight.device
            self._tokens = tokens
            self.residual = torch.empty(tokens, self.hidden, dtype=torch.bfloat16, device=dev)
            self.normed = torch.empty(tokens, self.hidden, dtype=torch.bfloat16, device=dev)

    def forward(self, x):
        """x BF16 [t, d] -> BF16 [t, d]: h <- h + moe(norm(h)) per block, final norm."""
        t = x.shape[0]
        self._reserve(t)
        residual, normed = self.residual[:t], self.normed[:t]
        residual.copy_(x)
        if t == 1 and self.one_launch:
            generations = tuple(layer.generation for layer in self.layers if hasattr(layer, "generation"))
            if self._fused is None or self._fused_generations != generations:
                first = self.layers[0]
                ex = first.experts
                blocks = [layer.block_descriptor(self.norm_weight) for layer in self.layers]
                from .layer import _group_of
                self._fused = StackDescriptor(blocks, ex.hidden_dim, ex.intermediate_dim, ex.local, first.n_shared,
                                              first.top_k, x.device, group=_group_of(first.device_mesh))
                self._fused_generations = tuple(layer.generation for layer in self.layers)
            self._fused.decode(x, self.layers[-1].partial[:1], residual, normed, self.eps)
            return normed
        normed.copy_(x)
        for layer in self.layers:
            add_rmsnorm(layer.forward_partial(normed), residual, self.norm_weight, self.eps, normed)
        return normed

    def launches_per_step(self) -> int:
        """Kernels of this library launched by one forward of one token batch <= 8."""
        if self.one_launch:
            return 1                  # the whole stack is one persistent kernel
        return 4 * len(self.layers)   # router+plan, gate/up, down, add+norm


class DecodeStackGraph:
    """Three eager warm-up steps on a side stream, then one captured graph of the whole
    stack; replay() runs it on the current contents of `self.token_in`."""

    def __init__(self, stack: MoEStack, example: torch.Tensor, capture: bool = True):
        self.stack = stack
        self.token_in = example.clone()
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream), torch.no_grad():
            for _ in range(3):
                self.out = stack(self.token_in)
        torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize()
        if torch.distributed.is_available() and torch.distributed.is_initialized():
            torch.distributed.barrier()
        self.graph = None
        if capture:
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=stream), torch.no_grad():
                self.out = stack(self.token_in)
        torch.cuda.synchronize()

    def replay(self) -> torch.Tensor:
        if self.graph is None:
            with torch.no_grad():
                self.out = self.stack(self.token_in)
        else:
            self.graph.replay()
        return self.out
