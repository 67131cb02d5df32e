"""SM partition on the GPU: the green-context ladder confines kernels to the SM count of the allowed-SM
mask (what SMPartitioner::SetStreamTpcMask achieves in the reference, common/sm_partition.cu:316-336),
and a training step that follows the mask computes the same step."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import resnet_oracle as O
from sirius_b200 import _runtime, ops  # noqa: F401
from sirius_b200._lib import call
from sirius_b200.step import ResNetStep

pytestmark = pytest.mark.gpu
FULL = (C.c_uint64 * 3)(2 ** 64 - 1, 2 ** 64 - 1, 2 ** 64 - 1)


def mask_of(n_sms):
    bits = (1 << n_sms) - 1
    return (C.c_uint64 * 3)(bits & (2 ** 64 - 1), (bits >> 64) & (2 ** 64 - 1), (bits >> 128) & (2 ** 64 - 1))


def levels():
    sms, n = (C.c_int * 32)(), C.c_int()
    call("srt_smp_partition_levels", 0, sms, 32, C.byref(n))
    return list(sms[:n.value])


def probe(stream_ptr):
    buf = torch.zeros(3, dtype=torch.int64, device="cuda")
    call("srt_debug_smid_probe", C.c_void_p(buf.data_ptr()), C.c_void_p(stream_ptr))
    torch.cuda.synchronize()
    return sum(bin(int(v) & (2 ** 64 - 1)).count("1") for v in buf.cpu().numpy().astype(np.uint64))


def test_ladder_and_confinement():
    total = torch.cuda.get_device_properties(0).multi_processor_count
    lv = levels()
    assert lv[0] == total and len(lv) >= 4
    assert all(a > b for a, b in zip(lv, lv[1:])) and lv[-1] >= 8
    own = torch.cuda.Stream()
    assert probe(own.cuda_stream) == total                   # an ordinary stream reaches every SM
    for allowed in (lv[1], lv[len(lv) // 2] + 3, lv[-1], 1):
        st, sms = C.c_void_p(), C.c_int()
        call("srt_smp_partition_stream", 0, allowed, C.byref(st), C.byref(sms))
        assert st.value is not None
        want = max([v for v in lv[1:] if v <= allowed], default=lv[-1])
        assert sms.value == want
        assert probe(st.value) == sms.value                  # the probe's blocks ran on exactly that many SMs
    st, sms = C.c_void_p(), C.c_int()
    call("srt_smp_partition_stream", 0, total, C.byref(st), C.byref(sms))
    assert st.value is None and sms.value == total           # whole device: keep your own stream


def test_step_follows_the_mask_and_computes_the_same_step():
    arch, B, IMG = "resnet14", 8, 64
    model = O.build_model(arch, 0)
    (im, lb), = O.make_batches(B, 1, IMG)
    lv = levels()
    try:
        ref = ResNetStep(layers=O.LAYERS[arch], max_batch=B, image=IMG, dtype="f32")
        ref.load_state_dict(O.state_arrays(model))
        ref.upload_batch(im, lb); ref.forward_backward(B, B); loss_ref = ref.loss()
        g_ref = ref.get("layer3.0.conv2.weight", 1)
        step = ResNetStep(layers=O.LAYERS[arch], max_batch=B, image=IMG, dtype="f32")
        step.load_state_dict(O.state_arrays(model))
        step.follow_sm_mask(True)
        for allowed in (lv[2] + 1, lv[-1], lv[0]):
            call("srt_set_sm_mask", mask_of(allowed))
            step.upload_batch(im, lb); step.forward_backward(B, B)
            loss = step.loss()
            want = lv[0] if allowed >= lv[0] else max(v for v in lv[1:] if v <= allowed)
            assert step.current_sms() == want
            g = step.get("layer3.0.conv2.weight", 1)
            # fewer SMs change the split of the filter-gradient sums, so equality is to rounding only
            assert abs(loss - loss_ref) <= 1e-5 * abs(loss_ref)
            assert np.abs(g - g_ref).max() <= 1e-4 * np.abs(g_ref).max()
        step.follow_sm_mask(False)
        step.upload_batch(im, lb); step.forward_backward(B, B)
        assert step.current_sms() == lv[0] and step.loss() == loss_ref
        assert ops.tc_status() == 0
        step.close(); ref.close()
    finally:
        call("srt_set_sm_mask", FULL)


def _transformer_cases():
    from oracle import gpt2_oracle as GO, qwen2_oracle as QO, swin_oracle as SO
    from sirius_b200.gpt2_step import Gpt2Step
    from sirius_b200.qwen2_step import Qwen2Step
    from sirius_b200.swin_step import SwinStep
    gcfg = dict(n_layer=2, n_head=4, d_model=128, vocab=500, ctx=64)
    qcfg = dict(n_layer=2, n_head=4, n_kv_head=2, hidden=128, intermediate=256, vocab=500)
    scfg = dict(image=224, patch=4, embed=32, depths=(2, 2, 2, 2), heads=(2, 4, 8, 16), window=7, num_classes=40)

    def gpt2():
        model = GO.build_model(**gcfg, seed=0)
        ids = GO.make_tokens(2, 64, gcfg["vocab"], 1)[0]
        mk = lambda: Gpt2Step(**gcfg, max_batch=2, seq=64)
        return mk, GO.state_arrays(model), (lambda s: s.upload_tokens(ids)), "transformer.h.1.mlp.c_fc.weight"

    def qwen2():
        model = QO.build_model(**qcfg, seed=0)
        ids = QO.make_tokens(2, 128, qcfg["vocab"], 1)[0]
        mk = lambda: Qwen2Step(**qcfg, max_batch=2, seq=128)
        return mk, QO.state_arrays(model), (lambda s: s.upload_tokens(ids)), "model.layers.1.mlp.down_proj.weight"

    def swin():
        model = SO.build_model(**scfg, seed=0)
        im, lb = SO.make_batches(2, 1, scfg["image"], scfg["num_classes"])[0]
        mk = lambda: SwinStep(**scfg, max_batch=2)
        return mk, SO.state_arrays(model), (lambda s: s.upload_batch(im.contiguous(), lb.contiguous())), \
            "features.5.1.mlp.0.weight"
    return {"gpt2": gpt2, "qwen2": qwen2, "swin": swin}


@pytest.mark.parametrize("which", ["gpt2", "qwen2", "swin"])
def test_transformer_executors_follow_the_mask_between_layers(which):
    """The GPT-2, Qwen2 and Swin executors move to the green-context partition that fits the allowed-SM mask
    between layers (main stream and the weight-gradient stream together), report its width, compute the same
    step there (to rounding: the filter-gradient split follows the SM count), and return to their own streams."""
    mk, state, upload, probe_name = _transformer_cases()[which]()
    lv = levels()
    GRAD = 1
    try:
        ref = mk()
        ref.load_state_dict(state)
        upload(ref); ref.forward_backward(); loss_ref = ref.loss()
        g_ref = ref.get(probe_name, GRAD)
        step = mk()
        step.load_state_dict(state)
        assert step.current_sms() == lv[0]
        step.follow_sm_mask(True)
        for allowed in (lv[2] + 1, lv[-1], lv[0]):
            call("srt_set_sm_mask", mask_of(allowed))
            upload(step); step.forward_backward()
            loss = step.loss()
            want = lv[0] if allowed >= lv[0] else max(v for v in lv[1:] if v <= allowed)
            assert step.current_sms() == want, (allowed, step.current_sms(), want)
            g = step.get(probe_name, GRAD)
            assert abs(loss - loss_ref) <= 1e-3 * abs(loss_ref)
            assert np.linalg.norm(g - g_ref) <= 1e-2 * np.linalg.norm(g_ref)
        call("srt_set_sm_mask", mask_of(lv[-1]))
        step.follow_sm_mask(False)                                   # back on the whole device whatever the mask says
        upload(step); step.forward_backward()
        assert step.current_sms() == lv[0] and step.loss() == loss_ref
        step.optimizer_step()
        step.synchronize()
        assert ops.tc_status() == 0
        step.close(); ref.close()
    finally:
        call("srt_set_sm_mask", FULL)
