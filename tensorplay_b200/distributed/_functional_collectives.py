"""Autograd-aware functional collectives and ``AsyncCollectiveTensor``
(tensorplay/distributed/_functional_collectives.py:174, 420-1040): PyTorch's implementation, plus the
reference's spellings of the single-tensor forms and the in-place point-to-point helpers."""
import torch
import torch.distributed as dist
from torch.distributed._functional_collectives import *  # noqa: F401,F403
from torch.distributed._functional_collectives import (AsyncCollectiveTensor, all_gather_into_tensor_coalesced,  # noqa: F401
                                                       all_gather_tensor, all_gather_tensor_autograd, all_reduce,
                                                       all_to_all_single, all_to_all_single_autograd,
                                                       reduce_scatter_tensor, reduce_scatter_tensor_autograd,
                                                       reduce_scatter_tensor_coalesced, wait_tensor)


def wait_tensors(tensors):
    return [wait_tensor(t) for t in tensors]


def all_gather_single(x, gather_dim, group, tag: str = ""):
    return all_gather_tensor(x, gather_dim, group, tag)


def all_gather_single_autograd(x, gather_dim, group, tag: str = ""):
    return all_gather_tensor_autograd(x, gather_dim, group, tag)


def reduce_scatter_single(x, reduce_op, scatter_dim, group, tag: str = ""):
    return reduce_scatter_tensor(x, reduce_op, scatter_dim, group, tag)


def reduce_scatter_single_autograd(x, reduce_op, scatter_dim, group, tag: str = ""):
    return reduce_scatter_tensor_autograd(x, reduce_op, scatter_dim, group, tag)


def all_gather_single_coalesced(tensors, group, tag: str = ""):
    return all_gather_into_tensor_coalesced(tensors, group, tag)


def reduce_scatter_single_coalesced(tensors, reduce_op, scatter_dims, group, tag: str = ""):
    return reduce_scatter_tensor_coalesced(tensors, reduce_op, scatter_dims, group, tag)


def reduce_scatter_inplace(output: torch.Tensor, input: torch.Tensor, op=dist.ReduceOp.SUM, group=None, async_op: bool = False):
    return dist.reduce_scatter_tensor(output, input, op=op, group=group, async_op=async_op)


def isend_inplace(tensor: torch.Tensor, dst: int, group=None, tag: int = 0):
    return dist.isend(tensor, dst, group=group, tag=tag)


def irecv_inplace(tensor: torch.Tensor, src: int, group=None, tag: int = 0):
    return dist.irecv(tensor, src, group=group, tag=tag)


def batch_p2p_ops_inplace(ops):
    """``ops``: list of ``(kind, tensor, peer)`` with kind "send" / "recv"; returns the work handles."""
    p2p = [dist.P2POp(dist.isend if k == "send" else dist.irecv, t, peer) for k, t, peer in ops]
    return dist.batch_isend_irecv(p2p) if p2p else []
