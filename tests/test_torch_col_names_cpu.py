"""The names training scripts and tools import from the reference's torch_col package exist here, under the same
module paths (torch_col, torch_col._C, torch_col._C._main, torch_col._C._dist, torch_col.xsched,
torch_col.util), and the ones that have a meaning without the reference's PyTorch fork do something."""
import io
import os
import uuid

import pytest
import torch

from sirius_b200 import torch_col as tc
from sirius_b200.torch_col import _C
from sirius_b200.torch_col._C import _dist, _main

TOP = """setup_colocate_training cleanup_colocate_training create_colocate_ctrl get_colocate_ctrl ColocateCtrl SwitchCtrl
DummyCtrl ColocateCtrlHookMode TrainMode ColocateAdjustL1Exception SwitchL1Exception EngineColocateAdjustL1Exception
register_saved_tensor_hook Trainer init_dynamic_batch DynamicBatchDataset MicroBatchManager BatchDistributePolicy
get_dynamic_dataset get_micro_batch_manager GradAccumulator MemoryPool EventManager info dinfo info_with_frame
DebugServer""".split()
MAIN = """is_configured is_enable_shared_tensor is_enable_dynamic_sm_partition is_enable_xsched get_colocate_ctrl_hook_mode
get_colocate_train_mode is_release_interm_memory_v1 is_release_interm_memory_v2 disable_release_interm_memory
disable_fbward_hook is_enable_fbward_hook is_train_master torch_col_init get_train_rank set_train_rank
get_train_world_size set_train_world_size set_train_rank_world_size has_colocated_infer_server
get_train_profile_log_path TorchColInit SMPartitionInit TorchDistExtInit cuda_memory_pool_infer_usage
cuda_memory_pool_train_usage cuda_memory_pool_train_peak_usage cuda_memory_pool_train_all_usage
cuda_memory_pool_free_train_local release_grad_fn_saved_tensor release_underlying_storage tag_model_start tag_model_end
tag_interm_memory release_interm_memory untag_interm_memory rearrange_memory DumpMempoolFreeList DumpMempoolBlockList
RegisterStream UnRegisterStream UnRegisterAllStreams GetXQueueSize GetXQueueSizeAllStreams GetTotalXQueueSize
AbortStream AbortAllStreams SyncStream SyncAllStreams SetRejectCudaCalls GuessNcclBegin GuessNcclEnd IsGuessNcclBegined
GetNcclStreams monitor_sm_partition CtrlEvent PyCtrlMsgEntry PyInfTraCommunicator init_train_info
update_current_batch_size get_unix_timestamp get_unix_timestamp_us CallGLOG_INFO CallGLOG_DINFO PyTensorWeakRef
PyDummyStub PySwitchStub PyColocateStub get_adjust_request_time_stamp get_adjust_done_time_stamp""".split()
DIST = """wait_barrier send_msg recv_msg _DynamicBatchDistirbutor init_dynamic_batch_distributor
init_train_performance_model _PerfModel Reducer ProcessGroupNCCL""".split()
XSCHED = """register_stream unregister_stream unregister_all_streams get_xqueue_size initial_kill_batch kill_batch
set_reject_cuda_calls guess_nccl_begin guess_nccl_end is_guess_nccl_begined get_nccl_streams""".split()


def test_every_name_of_the_reference_surface_is_present():
    missing = [n for n in TOP if not hasattr(tc, n)]
    missing += [f"_C._main.{n}" for n in MAIN if not hasattr(_main, n) or not hasattr(_C, n)]
    missing += [f"_C._dist.{n}" for n in DIST if not hasattr(_dist, n)]
    missing += [f"xsched.{n}" for n in XSCHED if not hasattr(tc.xsched, n)]
    assert hasattr(tc.util, "initialize_sgd_optimizer")
    assert not missing, missing
    for n in ("finalize_dropped_batch",):
        assert hasattr(_dist.Reducer, n)
    for n in ("_restart_nccl_comm", "_set_nccl_comm_abort_flag", "_set_as_default_pg"):
        assert hasattr(_dist.ProcessGroupNCCL, n)
    import sirius_b200.torch_col._C._main as m2     # the dotted import path of the reference's extension modules
    import sirius_b200.torch_col._C._dist as d2
    assert m2.get_train_rank is _C.get_train_rank and d2.wait_barrier is _C.dist.wait_barrier


def test_tensor_helpers_do_what_their_names_say():
    x = torch.randn(64, 32)
    w = _C.PyTensorWeakRef(x)
    assert w.nbytes() == 64 * 32 * 4 and w.storage_nbytes() >= w.nbytes() and w.data_ptr() == x.data_ptr()
    _C.release_underlying_storage(x)
    assert x.untyped_storage().nbytes() == 0 and w.storage_nbytes() == 0
    del x
    assert w.nbytes() == 0 and w.data_ptr() == 0                 # weak: the tensor is gone
    a = torch.randn(8, 8, requires_grad=True)
    loss = (a.exp() * a).sum()
    assert _C.release_grad_fn_saved_tensor(loss.grad_fn) == 0    # counts CUDA storage only; walks the graph without error


def test_names_without_a_counterpart_say_so():
    with pytest.raises(RuntimeError, match="not available"):
        _C.DumpMempoolFreeList("x")
    with pytest.raises(RuntimeError, match="not available"):
        _C.DumpMempoolBlockList("x")
    with pytest.raises(RuntimeError, match="deprecated"):
        _C.rearrange_memory()
    _dist.set_default_exchange(None)
    with pytest.raises(RuntimeError, match="not available"):
        _dist.ProcessGroupNCCL._restart_nccl_comm()
    assert _dist.Reducer.finalize_dropped_batch() is None
    assert _C.GetXQueueSize() == 0 and _C.GetNcclStreams() == [] and _C.IsGuessNcclBegined() is False


def test_monitor_sm_partition_prints_the_board(monkeypatch):
    """With a (debug) inference server holding 27 of 74 TPCs the monitor prints what the pre-launch hook would
    compute: 47 TPCs for training and the mask of the 27 closed ones."""
    name = f"srt_names_comm_{os.getpid()}_{uuid.uuid4().hex[:6]}"
    monkeypatch.setenv("COLTRAIN_HAS_INFER_SERVER", "1")
    monkeypatch.setenv("SIRIUS_B200_COMM_NAME", name)
    monkeypatch.setenv("SIRIUS_B200_DIST_NAME", name + "_dist")
    srv = tc.DebugServer(1, name)
    try:
        _C.torch_col_init(0, 1)
        srv.comm.infer_tpc(0, 1, 27)                              # AddInferRequiredTpcNum(27)
        buf = io.StringIO()
        _C.monitor_sm_partition(0.0, iterations=2, out=buf)
        lines = buf.getvalue().strip().splitlines()
        assert len(lines) == 2 and lines[0] == f"Infer TPC Num: 27, Train TPC Num: 47, Train Avail TPC Mask: {hex((1 << 27) - 1)}"
    finally:
        _C.torch_col_shutdown()
        srv.close()


def test_forward_and_backward_hooks_end_a_micro_batch_of_a_torch_module(monkeypatch):
    """ColocateCtrl.register_pytorch_hook on a torch.nn.Module (colocate_ctrl.py:101-110, 355-400): every leaf module
    checks the stub's command after its forward and before its backward; an L1 adjust raises
    ColocateAdjustL1Exception there, anything else lets the pass run. Step objects in the list are skipped."""
    import torch
    from sirius_b200.torch_col.colocate_ctrl import ColocateAdjustL1Exception, CtrlBase
    name = f"srt_hooks_{os.getpid()}_{uuid.uuid4().hex[:6]}"
    monkeypatch.setenv("COLTRAIN_HAS_INFER_SERVER", "1")
    monkeypatch.setenv("SIRIUS_B200_COMM_NAME", name)
    monkeypatch.setenv("SIRIUS_B200_DIST_NAME", name + "_dist")
    srv = tc.DebugServer(1, name)
    ctrl = None
    try:
        _C.torch_col_init(0, 1)
        ctrl = tc.create_colocate_ctrl(tc.TrainMode.COLOCATE_L1, tc.ColocateCtrlHookMode.XSCHED_SYNC, 1, 4)
        net = torch.nn.Sequential(torch.nn.Linear(8, 8), torch.nn.ReLU(), torch.nn.Sequential(torch.nn.Linear(8, 2)))
        ctrl.register_pytorch_hook([net, object()])
        x = torch.randn(4, 8, requires_grad=True)
        net(x).sum().backward()                                            # no command: nothing happens
        assert x.grad is not None
        # a command arriving after the second leaf's forward ends the forward pass there
        seen = []

        def command_arrives(m, i, o):
            seen.append("relu")
            ctrl._stub.cmd = _C.CtrlEvent.kColocateAdjustL1

        def last_layer_ran(m, i, o):
            seen.append("last")

        net[1].register_forward_hook(command_arrives)
        net[2][0].register_forward_hook(last_layer_ran)
        with pytest.raises(ColocateAdjustL1Exception, match="xsched_sync_fwd"):
            net(x)
        assert seen == ["relu"]                                            # the last layer's forward is reached, its own
        #                                                                    hook (registered first) raises before ours
        ctrl._stub.cmd = None
        # ... and one arriving between forward and backward ends the backward pass at its first leaf
        net2 = torch.nn.Sequential(torch.nn.Linear(8, 8), torch.nn.Tanh(), torch.nn.Linear(8, 1))
        ctrl.register_pytorch_hook([net2])
        y = net2(torch.randn(4, 8, requires_grad=True)).sum()
        ctrl._stub.cmd = _C.CtrlEvent.kColocateAdjustL1
        with pytest.raises(ColocateAdjustL1Exception, match="xsched_sync_bwd"):
            y.backward()
        ctrl._stub.cmd = _C.CtrlEvent.kColocateAdjustL2                    # not a kill command in this mode
        net2(torch.randn(4, 8)).sum().backward()
        _C.disable_fbward_hook()
        net3 = torch.nn.Linear(2, 2)
        ctrl.register_pytorch_hook([net3])
        assert len(net3._forward_hooks) == 0
    finally:
        _C._Config.use_fbward_hook = True
        if ctrl is not None:
            CtrlBase._reset()
        _C.torch_col_shutdown()
        srv.close()
