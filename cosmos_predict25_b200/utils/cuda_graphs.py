"""CUDA-graph capture of forward callables (launch-bound inner loops replay as one graph launch).

Parity target: the forward-only graph helper of the reference
(cosmos_predict2/_src/imaginaire/utils/graph.py:38-417: ``set_capture_start`` / ``is_graph_capturing`` /
``graph_pool_handle`` / ``make_graphed_callables_forward`` / ``create_cuda_graph``), which is a TransformerEngine-flavoured
variant of ``torch.cuda.make_graphed_callables``. This version has no TransformerEngine dependency: a callable is
warmed up on a side stream, captured once per input signature into a ``torch.cuda.CUDAGraph`` with static input and
output buffers, and replayed with a copy-in of the tensor arguments.

What can be captured: everything that launches on the current stream with arguments that do not change between
replays. The kernels of this package qualify (tensor maps are kernel parameters built from the static buffers'
addresses); the peer-memory barrier does not (its epoch is a launch argument that must advance on every call), so
callables that exchange data over a context-parallel group are run eagerly.
Non-tensor arguments (e.g. a RoPE table object) are treated as constants of the captured graph.
Without CUDA (CPU tests) every helper hands back the original callable.
"""

from __future__ import annotations

from typing import Any, Callable, Dict, Optional, Sequence, Tuple, Union

import torch
from torch.utils._pytree import tree_flatten, tree_unflatten

__all__ = ["GraphedForward", "make_graphed_callables_forward", "create_cuda_graph", "graph_pool_handle",
           "is_graph_capturing", "set_capture_start", "set_capture_end"]

_IS_GRAPH_CAPTURING = False


def set_capture_start() -> None:
    global _IS_GRAPH_CAPTURING
    _IS_GRAPH_CAPTURING = True


def set_capture_end() -> None:
    global _IS_GRAPH_CAPTURING
    _IS_GRAPH_CAPTURING = False


def is_graph_capturing() -> bool:
    """True while one of the helpers below is warming up or capturing (modules can skip host-side logging etc.)."""
    return _IS_GRAPH_CAPTURING


def graph_pool_handle():
    """Opaque id of a graph memory pool that several captures can share."""
    return torch.cuda.graph_pool_handle()


def _signature(flat) -> Tuple:
    return tuple((tuple(a.shape), a.dtype, a.device) if isinstance(a, torch.Tensor) else ("const", id(a)) for a in flat)


class GraphedForward:
    """``fn(*args, **kwargs)`` captured into a CUDA graph for one input signature (shapes, dtypes, devices).

    The call copies the tensor arguments into the static input buffers, replays the graph and returns the static
    outputs (valid until the next call; clone what must live longer). No autograd: call it under ``torch.no_grad``.
    """

    def __init__(self, fn: Callable, args: Sequence[Any], kwargs: Optional[Dict[str, Any]] = None, num_warmup_iters: int = 3,
                 pool=None):
        kwargs = dict(kwargs or {})
        flat, self._spec = tree_flatten((tuple(args), kwargs))
        self.signature = _signature(flat)
        self._static = [a.detach().clone() if isinstance(a, torch.Tensor) else a for a in flat]
        self._is_tensor = [isinstance(a, torch.Tensor) for a in flat]
        s_args, s_kwargs = tree_unflatten(self._static, self._spec)
        self.graph = torch.cuda.CUDAGraph()
        set_capture_start()
        try:
            with torch.no_grad():
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    for _ in range(num_warmup_iters):
                        fn(*s_args, **s_kwargs)
                torch.cuda.current_stream().wait_stream(side)
                torch.cuda.synchronize()
                with torch.cuda.graph(self.graph, pool=pool):
                    out = fn(*s_args, **s_kwargs)
        finally:
            set_capture_end()
        self._out_flat, self._out_spec = tree_flatten(out)

    def matches(self, args, kwargs) -> bool:
        flat, _ = tree_flatten((tuple(args), dict(kwargs or {})))
        return _signature(flat) == self.signature

    def __call__(self, *args, **kwargs):
        flat, _ = tree_flatten((tuple(args), kwargs))
        assert len(flat) == len(self._static), "argument structure differs from the captured call"
        for static, new, is_t in zip(self._static, flat, self._is_tensor):
            if is_t:
                assert static.shape == new.shape and static.dtype == new.dtype, "argument shape / dtype differs from the captured call"
                if static.data_ptr() != new.data_ptr():
                    static.copy_(new)
        self.graph.replay()
        return tree_unflatten(self._out_flat, self._out_spec)


def _cuda_in(flat) -> bool:
    return torch.cuda.is_available() and any(isinstance(a, torch.Tensor) and a.is_cuda for a in flat)


def make_graphed_callables_forward(modules: Union[Callable, Tuple[Callable, ...]],
                                   sample_args: Union[Tuple[Any, ...], Tuple[Tuple[Any, ...], ...]],
                                   num_warmup_iters: int = 3,
                                   sample_kwargs: Optional[Union[Dict[str, Any], Tuple[Dict[str, Any], ...]]] = None,
                                   pool=None) -> Union[Callable, Tuple[Callable, ...]]:
    """Forward-only graphed versions of ``modules`` (one callable or a tuple; ``sample_args`` / ``sample_kwargs`` follow
    the same structure). All captures share one memory pool, so graphing the blocks of a network in call order costs
    the activation memory of one block. CPU inputs: the callables come back unchanged."""
    single = not isinstance(modules, tuple)
    mods = (modules,) if single else modules
    s_args = (sample_args,) if single else sample_args
    s_kwargs = ((sample_kwargs or {}),) if single else (sample_kwargs or tuple({} for _ in mods))
    assert len(mods) == len(s_args) == len(s_kwargs)
    out = []
    shared_pool = pool
    for m, a, k in zip(mods, s_args, s_kwargs):
        flat, _ = tree_flatten((tuple(a), dict(k)))
        if not _cuda_in(flat):
            out.append(m)
            continue
        if shared_pool is None:
            shared_pool = graph_pool_handle()
        out.append(GraphedForward(m, a, k, num_warmup_iters, shared_pool))
    return out[0] if single else tuple(out)


def create_cuda_graph(cuda_graphs_storage: dict, blocks: torch.nn.ModuleList, x: torch.Tensor, emb: torch.Tensor,
                      context: torch.Tensor, rope=None, lora: Optional[torch.Tensor] = None,
                      extra_pos: Optional[torch.Tensor] = None, num_warmup_iters: int = 3) -> str:
    """Graph every DiT block for the shapes of this call (once per shape signature) and store the tuple of graphed blocks
    in ``cuda_graphs_storage`` under the returned key; ``storage[key][i](x, emb, context, rope, lora, extra_pos)`` then
    replays block i. Sample inputs are random tensors of the same shapes, as in the reference."""
    tensors = [t for t in (x, emb, context, lora, extra_pos) if t is not None]
    key = "_".join(str(d) for t in tensors for d in t.shape)
    if key not in cuda_graphs_storage:
        def dummy(t):
            return None if t is None else torch.randn(t.shape, device=t.device).to(t.dtype)
        sample = tuple((dummy(x), dummy(emb), dummy(context), rope, dummy(lora), dummy(extra_pos)) for _ in blocks)
        cuda_graphs_storage[key] = make_graphed_callables_forward(tuple(blocks), sample, num_warmup_iters=num_warmup_iters)
    return key
