"""torch_col: the Python surface the reference's training scripts import
(pytorch/torch_col/__init__.py:1-77), over the sirius_b200 runtime."""
from . import xsched  # noqa: F401
from ._C import *  # noqa: F401,F403
from ._C import (CtrlEvent, ColocateCtrlHookMode, TrainMode, PyCtrlMsgEntry, PyInfTraCommunicator, PyColocateStub,  # noqa: F401
                 PyDummyStub, PySwitchStub, dist, torch_col_init, torch_col_shutdown, set_train_step, get_train_step,
                 set_memory_pool, init_train_info, update_current_batch_size, get_train_rank, get_train_world_size,
                 is_train_master, is_configured, get_colocate_train_mode, get_colocate_ctrl_hook_mode,
                 is_enable_shared_tensor, is_enable_xsched, has_colocated_infer_server, get_unix_timestamp,
                 get_unix_timestamp_us, release_interm_memory, tag_model_start, tag_model_end)
from .util import MemoryPool, EventManager, info, dinfo, info_with_frame  # noqa: F401
from .accumulate import GradAccumulator  # noqa: F401
from .colocate_ctrl import (register_saved_tensor_hook, create_colocate_ctrl, get_colocate_ctrl, DummyCtrl,  # noqa: F401
                            SwitchCtrl, ColocateCtrl, SwitchL1Exception, ColocateAdjustL1Exception,
                            EngineColocateAdjustL1Exception)
from .trainer import Trainer  # noqa: F401
from .dynamic_batch import (DynamicBatchDataset, MicroBatchManager, get_dynamic_dataset, get_micro_batch_manager,  # noqa: F401
                            init_dynamic_batch, BatchDistributePolicy, DatasetType, VisionDatasetConfig,
                            TextDatasetConfig, Batch)
from .debug_server import DebugServer  # noqa: F401
from . import util  # noqa: F401


def setup_colocate_training(rank: int, world_size: int, will_use_nccl_comm: bool, init_nccl_process_group: bool):
    """__init__.py:31-66: runtime init, device selection, optional NCCL process group with a warm-up
    all-reduce. The training stream belongs to the step object, so no stream is created here."""
    import torch
    if init_nccl_process_group and not will_use_nccl_comm:
        raise ValueError('init_nccl_process_group is True but will_use_nccl_comm is False')
    torch_col_init(rank, world_size)
    if torch.cuda.is_available():
        torch.cuda.set_device(rank)
    if init_nccl_process_group:
        import torch.distributed as torch_dist
        if torch_dist.GroupMember.WORLD is not None:
            raise ValueError('torch.distributed already initialized')
        backend = "nccl" if torch.cuda.is_available() else "gloo"
        torch_dist.init_process_group(backend, rank=rank, world_size=world_size)
        ts = torch.tensor([42], device='cuda' if backend == "nccl" else 'cpu')
        torch_dist.all_reduce(ts)


def cleanup_colocate_training(destory_nccl_process_group: bool):
    xsched.unregister_all_streams()
    if destory_nccl_process_group:
        import torch.distributed as torch_dist
        torch_dist.destroy_process_group()
    from .colocate_ctrl import CtrlBase
    from .dynamic_batch import _reset_singletons
    CtrlBase._reset()
    _reset_singletons()
    torch_col_shutdown()
