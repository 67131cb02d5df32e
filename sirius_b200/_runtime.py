"""ctypes signatures of the host-side runtime entry points (include/sirius_runtime.h, sirius_pool.h)."""
from __future__ import annotations

import ctypes as C

from ._lib import register

_vp, _i, _i64, _u64, _d, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_uint64, C.c_double, C.c_size_t
_pi, _pd = C.POINTER(C.c_int), C.POINTER(C.c_double)


class CtrlMsg(C.Structure):
    _fields_ = [("id", _u64), ("event", _i), ("value", _i)]


class TrainInfo(C.Structure):
    _fields_ = [("train_pid", _i), ("train_rank", _i), ("train_world_size", _i), ("init_batch_size", _i),
                ("current_batch_size", _i), ("target_batch_size", _i), ("target_batch_size_unpublished", _i),
                ("model_name", C.c_char * 256), ("first_epoch_done", _i)]


class AdjusterConfig(C.Structure):
    _fields_ = [("base_mb", _d), ("slope_mb", _d), ("batch_size_limit", _i), ("enable_balance", _i),
                ("balance_threshold_mb", _d), ("num_visible_gpu", _i), ("use_shared_tensor", _i)]


class StubConfig(C.Structure):
    _fields_ = [("rank", _i), ("world_size", _i), ("kill_batch_on_recv", _i), ("is_colocate_l1", _i),
                ("input_batch_size", _i), ("poll_ms", _i), ("task_switch", _i)]


class PoolConfig(C.Structure):
    _fields_ = [("device", _i), ("backend", _i), ("page_nbytes", _sz), ("pool_nbytes", _sz),
                ("train_va_scale", _i), ("infer_va_scale", _i),
                ("unmap_on_release", _i)]


_PM, _PT = C.POINTER(CtrlMsg), C.POINTER(TrainInfo)
register({
    "srt_comm_open": (None, [C.c_char_p, _i, _i, _i, _i, C.POINTER(_vp)]),
    "srt_comm_close": (None, [_vp]),
    "srt_comm_world_size": (_i, [_vp]),
    "srt_comm_put": (None, [_vp, _PM, _i, _i]),
    "srt_comm_put_all": (None, [_vp, _PM, _i, _i]),
    "srt_comm_timed_get": (None, [_vp, _i, _i, _i, _PM, _pi]),
    "srt_comm_timed_get_from_any": (None, [_vp, _i, _i, _pi, _PM, _pi]),
    "srt_comm_clear": (None, [_vp]),
    "srt_comm_set_train_info": (None, [_vp, _i, _PT]),
    "srt_comm_get_train_info": (None, [_vp, _i, _PT]),
    "srt_comm_update_train_field": (None, [_vp, _i, _i, _i]),
    "srt_comm_get_train_field": (None, [_vp, _i, _i, _pi]),
    "srt_comm_invalidate_train_info": (None, [_vp, _i]),
    "srt_comm_infer_tpc": (None, [_vp, _i, _i, _i, _pi]),
    "srt_smp_train_avail_tpc_mask": (_u64, [_i, _i, _i, _i]),
    "srt_smp_train_avail_tpc_num": (_i, [_i, _i, _i, _i]),
    "srt_smp_allowed_sm_mask": (None, [_i, _i, _i, _i, C.POINTER(_u64)]),
    "srt_dist_open": (None, [C.c_char_p, _i, _i, _i, C.POINTER(_vp)]),
    "srt_dist_close": (None, [_vp]),
    "srt_dist_barrier": (None, [_vp, _i]),
    "srt_dist_send": (None, [_vp, _i, C.c_char_p, _i]),
    "srt_dist_recv": (None, [_vp, _i, C.c_char_p, _i, _i, _pi]),
    "srt_dist_switch_flag": (None, [_vp, _i, _i, _i, _pi]),
    "srt_dbd_init": (None, [_vp, _i, _i, _i, _i, _i]),
    "srt_dbd_distribute_batch": (None, [_vp, _vp, _i, _i, _i]),
    "srt_dbd_get_batch": (None, [_vp, _i, _pi, _i, _pi, _pi]),
    "srt_dbd_query_next_batch_size": (None, [_vp, _i, _pi]),
    "srt_dbd_finish_batch": (None, [_vp, _pi, _i, _i]),
    "srt_dbd_abort_batch": (None, [_vp, _pi, _i, _i]),
    "srt_dbd_vote_finish_last_micro_batch": (None, [_vp, _i, _pi]),
    "srt_dbd_vote_abort_last_micro_batch": (None, [_vp]),
    "srt_dbd_reset_last_micro_batch_finish_vote": (None, [_vp]),
    "srt_dbd_next_global_batch": (None, [_vp, _vp, _i]),
    "srt_dbd_next_epoch": (None, [_vp, _pi]),
    "srt_dbd_info": (None, [_vp, _i, _i, _pi]),
    "srt_perf_record_thpt": (None, [_vp, _i, _d]),
    "srt_perf_get_thpt": (None, [_vp, _i, _pd]),
    "srt_adjuster_create": (None, [_vp, C.POINTER(AdjusterConfig), C.POINTER(_vp)]),
    "srt_adjuster_destroy": (None, [_vp]),
    "srt_adjuster_load_train_info": (None, [_vp]),
    "srt_adjuster_reset_train_info": (None, [_vp]),
    "srt_adjuster_model_mem_param": (None, [C.c_char_p, _pd, _pd]),
    "srt_adjuster_model_mem_param_measured": (None, [C.c_char_p, _pd, _pd]),
    "srt_adjuster_predict_train_mem_mb": (None, [_vp, _i, _pd]),
    "srt_adjuster_infer_require_plan": (None, [_vp, _i, _d, _pd, _pi, _pi]),
    "srt_adjuster_infer_release_plan": (None, [_vp, _pd, _pd, _pd, _pi, _pi]),
    "srt_stub_set_abort_target": (None, [_vp, _vp, _vp]),
    "srt_stub_create": (None, [_vp, _vp, _vp, C.POINTER(StubConfig), C.POINTER(_vp)]),
    "srt_stub_stop": (None, [_vp]),
    "srt_stub_cmd": (_i, [_vp]),
    "srt_stub_set_cmd": (None, [_vp, _i]),
    "srt_stub_cmd_id": (_u64, [_vp]),
    "srt_stub_train_start": (None, [_vp]),
    "srt_stub_train_end": (None, [_vp]),
    "srt_stub_report_batch_size": (None, [_vp, _i]),
    "srt_stub_steps_no_interrupt_begin": (None, [_vp]),
    "srt_stub_steps_no_interrupt_end": (None, [_vp]),
    "srt_stub_adjust_l1_done": (None, [_vp]),
    "srt_stub_adjust_l2_done": (None, [_vp]),
    "srt_stub_target_batch_size": (None, [_vp, _i, _pi]),
    "srt_stub_set_killed_batch_recover": (None, [_vp]),
    "srt_stub_set_killed_batch_reconfiged": (None, [_vp]),
    "srt_stub_set_train_first_epoch_done": (None, [_vp]),
    "srt_stub_can_exit_after_infer_workload_done": (_i, [_vp]),
    "srt_stub_passed_ms_from_set_cmd": (_d, [_vp]),
    "srt_stub_try_interrupt_train_done": (None, [_vp, _i, _pi]),
    "srt_stub_prepare_resume": (None, [_vp, _pi]),
    "srt_stub_switch_flag": (None, [_vp, _i, _i, _i, _pi]),
    "srt_stub_adjust_timestamps": (_i, [_vp, _i, C.POINTER(_i64), _i]),
    "srt_pool_create": (None, [C.POINTER(PoolConfig), C.POINTER(_vp)]),
    "srt_pool_create_shared": (None, [C.POINTER(PoolConfig), C.c_char_p, C.POINTER(_vp)]),
    "srt_pool_attach": (None, [C.c_char_p, _i, _i, C.POINTER(_vp)]),
    "srt_pool_destroy": (None, [_vp]),
    "srt_pool_init": (None, [_i, _sz, _i]),
    "srt_pool_shutdown": (None, [_i]),
    "srt_pool_default": (None, [_i, C.POINTER(_vp)]),
    "srt_alloc": (_vp, [_sz, _i, _vp]),
    "srt_free": (C.c_void_p, [_vp, _sz, _i, _vp]),
    "srt_record_stream": (None, [_vp, _i, _vp]),
    "srt_empty_cache": (None, [_i, C.POINTER(_sz)]),
    "srt_tag_model_begin": (None, []),
    "srt_tag_model_end": (None, []),
    "srt_tag_interm": (None, [_vp, _i]),
    "srt_untag_interm": (None, [_i]),
    "srt_release_interm": (None, [_i, C.POINTER(_sz)]),
    "srt_pool_stat_dev": (_i64, [_i, _i]),
    "srt_alloc_counters": (None, [_i, C.POINTER(_i64), C.POINTER(_i64), C.POINTER(_i64), C.POINTER(_i64), C.POINTER(_i64)]),
    "srt_pool_alloc": (None, [_vp, _i, _sz, C.POINTER(_vp)]),
    "srt_pool_free": (None, [_vp, _i, _vp]),
    "srt_pool_hollow": (None, [_vp, _i, _vp]),
    "srt_pool_empty_cache": (None, [_vp, _i, C.POINTER(_sz)]),
    "srt_pool_stat": (_i64, [_vp, _i]),
    "srt_pool_set_oom_handler": (None, [_vp, _vp, _vp]),
    "srt_resnet_create_with_pool": (None, [_vp, _vp, C.POINTER(_vp)]),
    "srt_resnet_create_on_allocator": (None, [_vp, _vp, _i, C.POINTER(_vp)]),
    "srt_step_release_activations": (None, [_vp, C.POINTER(_sz)]),
    "srt_step_shrink_activations": (None, [_vp, C.c_int, C.POINTER(_sz)]),
    "srt_step_reserve_activations": (None, [_vp, _i]),
    "srt_step_request_abort": (None, [_vp, _i]),
    "srt_step_follow_sm_mask": (None, [_vp, _i]),
    "srt_step_overlap_wgrad": (None, [_vp, _i]),
    "srt_step_num_grad_buckets": (_i, [_vp]),
    "srt_step_grad_bucket": (None, [_vp, _i, C.POINTER(_i64), C.POINTER(_i64)]),
    "srt_step_wait_grad_bucket": (None, [_vp, _i, _vp]),
    "srt_step_wait_event": (None, [_vp, _vp]),
    "srt_step_current_sms": (None, [_vp, C.POINTER(_i)]),
    "srt_step_follow_infer_tpc": (None, [_vp, _vp, _i, _i, _i]),
    "srt_gpt2_follow_infer_tpc": (None, [_vp, _vp, _i, _i, _i, _i]),
    "srt_qwen2_follow_infer_tpc": (None, [_vp, _vp, _i, _i, _i, _i]),
    "srt_swin_follow_infer_tpc": (None, [_vp, _vp, _i, _i, _i, _i]),
    "srt_gpt2_current_sms": (_i, [_vp]),
    "srt_qwen2_current_sms": (_i, [_vp]),
    "srt_swin_current_sms": (_i, [_vp]),
    "srt_smp_partition_levels": (None, [_i, C.POINTER(_i), _i, C.POINTER(_i)]),
    "srt_smp_partition_stream": (None, [_i, _i, C.POINTER(_vp), C.POINTER(_i)]),
    "srt_debug_smid_probe": (None, [_vp, _vp]),
})
