"""Module paths of the reference keep importing: own files first, PyTorch's module of the same path next (as the
SAME module object, never a second execution of its source), views of the domain packs last."""
import importlib

import pytest


@pytest.mark.parametrize("name,torch_name", [
    ("distributed.tensor._ops._math_ops", "torch.distributed.tensor._ops._math_ops"),
    ("distributed.fsdp._fully_shard._fsdp_collectives", "torch.distributed.fsdp._fully_shard._fsdp_collectives"),
    ("distributed.elastic.rendezvous.etcd_store", "torch.distributed.elastic.rendezvous.etcd_store"),
    ("distributed._shard.sharded_tensor.api", "torch.distributed._shard.sharded_tensor.api"),
    ("distributed.algorithms.ddp_comm_hooks.ddp_zero_hook", "torch.distributed.algorithms.ddp_comm_hooks.ddp_zero_hook"),
    ("distributed.flight_recorder.components.types", "torch.distributed.flight_recorder.components.types"),
    ("nn.utils.rnn", "torch.nn.utils.rnn"),
    ("optim.lbfgs", "torch.optim.lbfgs"),
])
def test_paths_without_a_file_here_are_pytorchs_module_objects(name, torch_name):
    ours = importlib.import_module("tensorplay_b200." + name)
    assert ours is importlib.import_module(torch_name)


def test_own_modules_win_and_submodule_paths_exist():
    from tensorplay_b200.distributed.algorithms import ddp_comm_hooks as H
    from tensorplay_b200.distributed.algorithms.ddp_comm_hooks.default_hooks import allreduce_hook
    from tensorplay_b200.distributed.algorithms.ddp_comm_hooks.powerSGD_hook import PowerSGDState, powerSGD_hook
    from tensorplay_b200.distributed.algorithms.ddp_comm_hooks.post_localSGD_hook import PostLocalSGDState
    from tensorplay_b200.distributed.algorithms.model_averaging.averagers import PeriodicModelAverager
    from tensorplay_b200.distributed.algorithms.model_averaging.utils import average_parameters
    from tensorplay_b200.distributed.elastic.multiprocessing.errors import record
    from tensorplay_b200.distributed.optim import ZeroRedundancyOptimizer
    import tensorplay_b200.distributed.algorithms as A
    assert allreduce_hook is A.allreduce_hook and PostLocalSGDState is A.PostLocalSGDState
    assert H.powerSGD_hook.powerSGD_hook is powerSGD_hook and PowerSGDState(None, 2)["rank"] == 2
    assert PeriodicModelAverager.__module__.startswith("tensorplay_b200")
    assert ZeroRedundancyOptimizer.__module__ == "tensorplay_b200.distributed.optim.zero"
    assert average_parameters.__module__.startswith("tensorplay_b200") and callable(record)


def test_domain_pack_views():
    import tensorplay_b200.lumen as L
    import tensorplay_b200.metrics as M
    from tensorplay_b200.lumen._core.layer.grad_cam import LayerGradCam
    from tensorplay_b200.metrics.classification.accuracy import BinaryAccuracy
    from tensorplay_b200.metrics.functional.classification.accuracy import binary_accuracy
    from tensorplay_b200.metrics.text.bleu import BLEUScore
    assert BinaryAccuracy is M.BinaryAccuracy and BLEUScore is M.BLEUScore and LayerGradCam is L.LayerGradCam
    assert binary_accuracy is M.functional.binary_accuracy
    with pytest.raises(ImportError):
        from tensorplay_b200.metrics.classification.accuracy import NoSuchMetric  # noqa: F401


def test_alias_spelling_reaches_the_same_objects():
    import tensorplay_b200.compat as compat
    compat.install_alias()
    from tensorplay.distributed.elastic.multiprocessing.errors import record
    from tensorplay.metrics.regression.mse import MeanSquaredError
    from tensorplay.vision.ops import nms
    import tensorplay_b200.metrics as M
    from tensorplay_b200.distributed.elastic.multiprocessing import record as r0
    from tensorplay_b200.vision.ops import nms as n0
    assert record is r0 and MeanSquaredError is M.MeanSquaredError and nms is n0


def test_linalg_sparse_func_additions():
    import torch
    import tensorplay_b200 as tp
    torch.manual_seed(0)
    A = torch.randn(6, 4, dtype=torch.float64)
    U, P = tp.linalg.polar(A)
    assert torch.allclose(U @ P, A) and torch.allclose(U.mH @ U, torch.eye(4, dtype=torch.float64))
    assert torch.allclose(P, P.mH) and torch.linalg.eigvalsh(P).min() > -1e-12
    U2, P2 = tp.linalg.polar(A.T, side="left")
    assert torch.allclose(P2 @ U2, A.T)
    S = A.T @ A
    R = tp.linalg.matrix_sqrth(S)
    assert torch.allclose(R @ R, S) and torch.allclose(R, R.mH)
    z = torch.randn(5, dtype=torch.complex128)
    assert torch.allclose(tp.linalg.vdot(z, z), (z.conj() * z).sum()) and tp.linalg.svd is torch.linalg.svd
    sp = torch.tensor([[4.0, 1.0], [1.0, 3.0]]).to_sparse()
    b = torch.tensor([1.0, 2.0])
    assert torch.allclose(sp.to_dense() @ tp.sparse.solve(sp, b), b)
    assert tp.sparse.sparse_coo_tensor is torch.sparse_coo_tensor and tp.sparse.to_dense(sp).shape == (2, 2)
    x = torch.randn(7, 4)
    assert torch.allclose(tp.func.chunk_vmap(lambda r: r.sin().sum(), chunks=3)(x), x.sin().sum(1))
    assert tp.func.rearrange(torch.arange(6).view(2, 3), "a b -> b a").shape == (3, 2)
    net = torch.nn.Sequential(torch.nn.Linear(3, 3), torch.nn.BatchNorm1d(3))
    tp.func.batch_norm_without_running_stats(net)
    assert net[1].running_mean is None and not net[1].track_running_stats
    import tensorplay_b200.graph.passes as gp
    assert gp is importlib.import_module("torch.fx.passes")
    from tensorplay_b200.nn.modules import BatchNorm2d, GatedDeltaNet  # PyTorch's long tail next to own layers
    assert BatchNorm2d is torch.nn.BatchNorm2d and GatedDeltaNet.__module__.startswith("tensorplay_b200")


def test_fallback_packages_show_pytorchs_names_and_the_references_extras():
    import torch
    import tensorplay_b200 as tp
    import tensorplay_b200.export as E
    import tensorplay_b200.export.graph_signature as gs
    import tensorplay_b200.graph as G
    assert E is tp.export and E.Dim is torch.export.Dim and E.InputKind is torch.export.graph_signature.InputKind
    assert gs is importlib.import_module("torch.export.graph_signature")          # same object, not a second execution
    assert G.symbolic_trace is torch.fx.symbolic_trace and G.TensorType is torch.fx.tensor_type.TensorType
    assert importlib.import_module("tensorplay_b200.graph.passes") is importlib.import_module("torch.fx.passes")
    assert tp.accelerator.Graph is torch.cuda.CUDAGraph and tp.monitor.StatResult._fields[0] == "name"
    with pytest.raises(AttributeError):
        tp.export.no_such_name


def test_backends_package():
    import torch
    import tensorplay_b200 as tp
    assert tp.backends.cudnn is torch.backends.cudnn and tp.backends.cuda.matmul is torch.backends.cuda.matmul
    assert tp.backends.cuda.is_available() == torch.cuda.is_available() and not tp.backends.cuda.is_ck_sdpa_available()
    assert tp.backends.cuda.get_name() == (torch.cuda.get_device_name() if torch.cuda.is_available() else "cpu")
    assert importlib.import_module("tensorplay_b200.backends.cudnn") is torch.backends.cudnn

