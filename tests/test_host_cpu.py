"""CPU-only checks of the host side: the C-ABI library loads and exports every declared symbol,
argument validation happens before any launch, and the Python mirror of the reference's
interface (config tree, maps, optimizer constructors, enable rule) behaves like the reference."""
import ctypes
import os
import pickle
import re

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from lpmm import _native as N
    header = open(os.path.join(ROOT, "include", "lpmm_b200.h")).read()
    declared = set(re.findall(r"\b(lpmm_b200_[a-z0-9_]+)\s*\(", header))
    assert len(declared) >= 19
    lib = ctypes.CDLL(N._LIB_PATH)
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in include/lpmm_b200.h but not exported"
    assert declared == set(N.SIGNATURES), "the ctypes table and the header disagree"
    assert N.lib.lpmm_b200_abi_version() == 3
    # and nothing else under the library's prefix is exported: helpers shared between its translation units stay hidden
    import shutil
    import subprocess
    if shutil.which("nm"):
        out = subprocess.run(["nm", "-D", "--defined-only", N._LIB_PATH], capture_output=True, text=True).stdout
        exported = set(re.findall(r" T (lpmm_b200_[a-z0-9_]+)", out))
        assert exported == declared, f"exported but not declared: {sorted(exported - declared)}"


def test_argument_validation_without_a_gpu():
    from lpmm import _native as N
    lib = N.lib
    assert lib.lpmm_b200_strerror(0) == b"ok"
    assert lib.lpmm_b200_packed_len(1) == 1025 and lib.lpmm_b200_packed_len(2048) == 1025
    assert lib.lpmm_b200_packed_len(2049) == 2049 and lib.lpmm_b200_packed_len(0) == 1
    assert lib.lpmm_b200_packed_len(-1) == -2
    assert lib.lpmm_b200_pack_nonlinear4(None, 7, None, None, None) == -2      # odd count
    assert lib.lpmm_b200_pack_nonlinear4(None, 8, None, None, None) == -1      # null pointers
    assert lib.lpmm_b200_adamw4bit_multi_tensor(None, -1, None, None, N.Hyper(), 0, -1, None) == -2
    arr = (N.Tensor * 2)()
    arr[0] = N.Tensor(0, 0, 0, 0, 0, 0, 300, N.KIND_Q4, 0)
    arr[1] = N.Tensor(0, 0, 0, 0, 0, 0, 4096, N.KIND_FP32, 0)
    assert lib.lpmm_b200_count_groups(arr, 2) == 3 + 32
    assert lib.lpmm_b200_adamw4bit_multi_tensor(arr, 2, None, None, N.Hyper(), 0, -1, None) == -1  # null data
    arr[0].kind = 7
    assert lib.lpmm_b200_adamw4bit_multi_tensor(arr, 2, None, None, N.Hyper(), 0, -1, None) == -3
    shape = (ctypes.c_int64 * 3)(2, 100, 64)
    tiles = (100 + 63) // 64
    assert lib.lpmm_b200_factored_scratch_bytes(shape, 3) == 4 * (2 * tiles * 64 + 2)
    assert lib.lpmm_b200_factored_scratch_bytes(shape, 1) == -2
    # code widths and group sizes
    assert lib.lpmm_b200_packed_len_bits(2049, 4) == 2049 and lib.lpmm_b200_packed_len_bits(2049, 8) == 4097
    assert lib.lpmm_b200_packed_len_bits(10, 3) == -5 and lib.lpmm_b200_packed_len_bits(10, 9) == -3
    assert lib.lpmm_b200_quant_group(None, 10, None, 4, 100, None, None, None) == -5      # not a power of two
    assert lib.lpmm_b200_quant_group(None, 10, None, 4, 8192, None, None, None) == -5     # larger than 4096
    assert lib.lpmm_b200_quant_group(None, 10, None, 4, 256, None, None, None) == -1      # null pointers
    assert lib.lpmm_b200_pack_nonlinear(None, 7, None, 8, None, None) == -1               # odd counts are fine for bytes
    # list entry points
    assert lib.lpmm_b200_adamw4bit_unfused_step_many(None, -1, None, None, 0.9, 0.999, 1e-3, 0.0, 1e-8, None, None, 0,
                                                     None) == -2
    assert lib.lpmm_b200_adamw4bit_unfused_step_many(None, 2, None, None, 0.9, 0.999, 1e-3, 0.0, 1e-8, None, None, 0,
                                                     None) == -1
    assert lib.lpmm_b200_adamw4bit_unfused_step_many(None, 0, None, None, 0.9, 0.999, 1e-3, 0.0, 1e-8, None, None, 0,
                                                     None) == 0
    arr[0].kind = N.KIND_Q4
    offs = (ctypes.c_int64 * 9)(*([32] * 9))
    assert lib.lpmm_b200_adamw4bit_multi_tensor_zero1(arr, 2, None, None, N.Hyper(), 0, -1, offs, 8, offs, 2, 0.5, None) == -2
    assert lib.lpmm_b200_adamw4bit_multi_tensor_zero1(arr, 2, None, None, N.Hyper(), 0, -1, offs, 1, offs, 9, 0.5, None) == -2
    assert lib.lpmm_b200_adamw4bit_multi_tensor_zero1(arr, 2, None, None, N.Hyper(), 0, -1, offs, 1, None, 2, 0.5, None) == -1
    assert lib.lpmm_b200_sgd4bit_multi_tensor(arr, 2, None, 0.0, 0.0, 1e-2, 0.0, 0, 0, 0, -1, None) == -3  # momentum 0
    assert lib.lpmm_b200_sgd4bit_multi_tensor(arr, 2, None, 0.0, 0.9, 1e-2, 0.0, 0, 0, 0, -1, None) == -1  # null data
    assert lib.lpmm_b200_sgd4bit_multi_tensor(None, -1, None, 0.0, 0.9, 1e-2, 0.0, 0, 0, 0, -1, None) == -2


def test_maps_are_the_reference_maps(qmaps):
    from lpmm.functional import create_general_qmap
    assert np.array_equal(create_general_qmap("nonlinear", 4, True).numpy(), qmaps["m"])
    assert np.array_equal(create_general_qmap("power-1", 4, False).numpy(), qmaps["v"])
    assert np.array_equal(create_general_qmap("nonlinear", 4, False).numpy(), qmaps["nonlinear_unsigned"])
    assert np.array_equal(create_general_qmap("power-2", 4, False).numpy(), qmaps["power2"])
    assert np.array_equal(create_general_qmap("power-1", 4, True).numpy(), qmaps["power1_signed"])
    assert create_general_qmap("linear", 4, True) is None
    with pytest.raises(ValueError):
        create_general_qmap("no-such-map", 4, True)
    for b in (5, 6, 7, 8):  # the maps of default_{5,6,7,8}b.yml
        assert np.array_equal(create_general_qmap("nonlinear", b, True).numpy(), qmaps[f"nonlinear_{b}"])
        assert np.array_equal(create_general_qmap("power-1", b, False).numpy(), qmaps[f"power1_{b}"])
        assert np.all(np.diff(qmaps[f"nonlinear_{b}"]) > 0) and len(qmaps[f"nonlinear_{b}"]) == 1 << b


def test_config_defaults_files_and_pickle(tmp_path):
    from lpmm.config import CONFIG_DIR, get_config
    c = get_config(None)
    assert (c.QUANT.M.BITS, c.QUANT.M.SCALE_TYPE.DEFAULT, c.QUANT.M.QUANT_TYPE.DEFAULT, c.QUANT.M.SIGNED) == (4, "group", "nonlinear", True)
    assert (c.QUANT.SQM.SCALE_TYPE.DEFAULT, c.QUANT.SQM.QUANT_TYPE.DEFAULT, c.QUANT.SQM.SIGNED) == ("group", "power-1", False)
    assert c.QUANT.M.THRESHOLD == 4096 and c.QUANT.M.ROUND_TYPE == "real-nearest" and c.QUANT.M.GROUP_SIZE == 128
    d = get_config(os.path.join(CONFIG_DIR, "default.yml"))
    assert d.QUANT.SQM.SCALE_TYPE.DEFAULT == "rank1" and d.QUANT.SQM.SIGNED is False and d.QUANT.M.ENABLE is True
    assert pickle.loads(pickle.dumps(d)) == d
    with pytest.raises(AttributeError):
        d.QUANT.M.BITS = 8                                       # frozen
    base = tmp_path / "base.yml"
    base.write_text("QUANT:\n  M:\n    ENABLE: false\n")
    child = tmp_path / "child.yml"
    child.write_text("BASE: ['base.yml']\nQUANT:\n  SQM:\n    SCALE_TYPE:\n      DEFAULT: rank1\n")
    e = get_config(str(child))
    assert e.QUANT.M.ENABLE is False and e.QUANT.SQM.SCALE_TYPE.DEFAULT == "rank1"
    with pytest.raises(TypeError):
        get_config(123)
    assert not os.path.exists("lpmm_config.txt")


def test_optimizer_constructors_validate_like_the_reference():
    import lpmm
    w = torch.nn.Parameter(torch.zeros(8, 8))
    for bad in (dict(lr=-1.0), dict(eps=-1.0), dict(betas=(1.0, 0.9)), dict(betas=(0.9, -0.1)), dict(weight_decay=-1.0)):
        with pytest.raises(ValueError):
            lpmm.optim.AdamW([w], **bad)
    # fused=True, which the reference's SGD rejects (sgd.py:31-32), is accepted here and leaves the
    # param_group keys (hence the state_dict) as they are without it
    assert (lpmm.optim.SGD([w], lr=0.1, fused=True).state_dict()["param_groups"][0].keys()
            == lpmm.optim.SGD([w], lr=0.1).state_dict()["param_groups"][0].keys())
    with pytest.raises(ValueError):
        lpmm.optim.SGD([w], lr=-0.1)
    opt = lpmm.optim.AdamW([w], fused=True)
    assert opt.defaults["fused"] is True and opt.qconfig.QUANT.M.BITS == 4
    assert set(opt.state_dict()) >= {"state", "param_groups", "qconfig"}


def test_fused_rank1_option_applies_only_to_rank1_configurations():
    """fused_rank1 is an extension that is off by default; it takes effect only for a 4-bit rank-1 second
    moment without factorisation, and says so for wider codes instead of silently changing the layout."""
    import os
    import lpmm
    from lpmm.config import CONFIG_DIR
    w = torch.nn.Parameter(torch.zeros(8, 8))
    cfg = lambda n: os.path.join(CONFIG_DIR, n)
    opt = lpmm.optim.AdamW([w], fused=True)
    assert opt._fused_rank1 is False and not opt._fused_rank1_applies(opt.param_groups[0])
    opt = lpmm.optim.AdamW([w], fused=True, fused_rank1=True, qconfig=cfg("default.yml"))
    assert opt._fused_rank1_applies(opt.param_groups[0])
    assert "fused_rank1" not in opt.state_dict()["param_groups"][0]  # param_group keys stay the reference's
    opt = lpmm.optim.AdamW([w], fused=True, fused_rank1=True, qconfig=cfg("default.yml"), factor_second_moment=True)
    assert not opt._fused_rank1_applies(opt.param_groups[0])
    opt = lpmm.optim.AdamW([w], fused=True, fused_rank1=True)  # group scales: the fused kernel holds them itself
    assert not opt._fused_rank1_applies(opt.param_groups[0])
    opt = lpmm.optim.AdamW([w], fused=True, fused_rank1=True, qconfig=cfg("default_8b.yml"))
    if opt.get_qmetadata_by_state_name("exp_avg_sq")["scale_type"] == "rank1":
        with pytest.raises(NotImplementedError):
            opt._fused_rank1_applies(opt.param_groups[0])


def test_fused_arith_entry_points_refuse_what_they_do_not_cover():
    """The fused arithmetic on non-fused states: 4-bit codes only, no factored second moment, moments both fp32
    or both quantized -- refused before any CUDA call."""
    from lpmm import _native as N
    one = N.lib.lpmm_b200_adamw4bit_fused_arith_step
    many = N.lib.lpmm_b200_adamw4bit_fused_arith_step_many
    hp = (0.9, 0.999, 1e-3, 0.01, 1e-8)
    t = N.StepTensor()
    t.numel, t.ndim = 0, 2
    t.shape[0], t.shape[1] = 0, 8
    t.m_mode, t.v_mode = N.STATE_GROUP4, N.STATE_RANK1_4
    assert one(ctypes.byref(t), None, None, *hp, 1.0, None) == 0          # empty tensor: nothing to do
    t.m_bits = t.v_bits = 8
    assert one(ctypes.byref(t), None, None, *hp, 1.0, None) == -5         # wider codes
    t.m_bits = t.v_bits = 4
    t.v_mode = N.STATE_FACTORED
    assert one(ctypes.byref(t), None, None, *hp, 1.0, None) == -5         # factored second moment
    t.m_mode, t.v_mode = N.STATE_FP32, N.STATE_GROUP4
    assert one(ctypes.byref(t), None, None, *hp, 1.0, None) == -5         # mixed fp32 / quantized moments
    assert one(None, None, None, *hp, 1.0, None) == -1
    assert many(None, -1, None, None, *hp, None, None, 0, None) == -2
    assert many(None, 2, None, None, *hp, None, None, 0, None) == -1
    assert many(None, 0, None, None, *hp, None, None, 0, None) == 0


def test_fused_16bit_entry_point_argument_checks():
    """Argument errors of the bf16 / fp16 step are found before any CUDA call."""
    from lpmm import _native as N
    h = N.Hyper(0.9, 0.999, 1e-3, 0.01, 1e-8, 1.0)
    arr = (N.Tensor * 1)()
    fn = N.lib.lpmm_b200_adamw4bit_multi_tensor_16bit
    assert fn(arr, 0, 7, None, None, h, 0, -1, None) == -3           # unknown element type
    assert fn(arr, 0, N.DTYPE_BF16, None, None, h, 0, -1, None) == 0  # an empty list is a no-op
    assert fn(None, 1, N.DTYPE_FP16, None, None, h, 0, -1, None) == -1
    assert fn(arr, 0, N.DTYPE_FP16, None, None, h, 0, 5, None) == -2  # range beyond the list


def test_enable_rule_and_override():
    import lpmm
    from lpmm.optim.optimizer import quantize_enabled
    assert quantize_enabled(torch.zeros(4097), True, 4096) is True
    assert quantize_enabled(torch.zeros(4096), True, 4096) is False          # exactly the threshold stays fp32
    assert quantize_enabled(torch.zeros(10 ** 5), False, 4096) is False
    lin = torch.nn.Linear(128, 64)
    opt = lpmm.optim.AdamW(lin.parameters())
    opt.override_quantize_enable(lin, "weight", False)
    assert opt.override_q_enable[id(lin.weight)] is False
    opt.state[lin.weight]["step"] = torch.tensor(1.0)
    with pytest.raises(ValueError):
        opt.override_quantize_enable(lin, "weight", True)


def test_cpu_tensors_are_rejected_not_silently_computed():
    """There is no CPU implementation: a step on CPU tensors raises like the reference's bindings do."""
    import lpmm
    w = torch.nn.Parameter(torch.randn(100, 50))
    w.grad = torch.randn(100, 50)
    for kw in (dict(fused=True), dict(fused=False), dict(factor_second_moment=True)):
        opt = lpmm.optim.AdamW([w], **kw)
        with pytest.raises(RuntimeError):
            opt.step()
    opt = lpmm.optim.SGD([w], lr=0.1, momentum=0.9)
    with pytest.raises(RuntimeError):
        opt.step()


def test_flags_entry_points_validate_without_a_gpu():
    """The ..._flags / ..._16bit_peers entry points refuse unknown flags, bad peer counts and unaligned offsets before
    anything is launched."""
    import ctypes
    from lpmm import _native as N
    t = (N.Tensor * 1)(N.Tensor(0x1000, 0x2000, 0x3000, 0x4000, 0x5000, 0x6000, 256, N.KIND_Q4, 0))
    h = N.Hyper(0.9, 0.999, 1e-3, 0.01, 1e-8, 1.0)
    qm = ctypes.c_void_p(0x7000)
    assert N.lib.lpmm_b200_adamw4bit_multi_tensor_flags(t, 1, qm, qm, h, 0, -1, 4, None) == -3
    assert N.lib.lpmm_b200_adamw4bit_multi_tensor_flags(t, 1, None, None, h, 0, -1, 1, None) == -1
    assert N.lib.lpmm_b200_adamw4bit_multi_tensor_flags(t, 1, qm, qm, h, 0, 0, 1, None) == 0  # empty range: nothing to do
    assert N.lib.lpmm_b200_adamw4bit_multi_tensor_flags(t, 1, qm, qm, h, 1, 5, 1, None) == -2
    offs = (ctypes.c_int64 * 2)(64, 8)
    assert N.lib.lpmm_b200_adamw4bit_multi_tensor_16bit_peers(t, 1, N.DTYPE_BF16, qm, qm, h, 0, -1, offs, 9, 0, None) == -2
    assert N.lib.lpmm_b200_adamw4bit_multi_tensor_16bit_peers(t, 1, N.DTYPE_BF16, qm, qm, h, 0, -1, offs, 2, 0, None) == -2
    assert N.lib.lpmm_b200_adamw4bit_multi_tensor_16bit_peers(t, 1, N.DTYPE_BF16, qm, qm, h, 0, -1, None, 2, 0, None) == -1
    assert N.lib.lpmm_b200_adamw4bit_multi_tensor_16bit_peers(t, 1, 7, qm, qm, h, 0, -1, offs, 1, 0, None) == -3
    assert N.lib.lpmm_b200_adamw4bit_multi_tensor_peers_flags(t, 1, qm, qm, h, 0, -1, offs, 2, 0, None) == -2  # 8 % 32 != 0
    # the list forms of the non-fused step: unknown flag bits refused, an empty list is a no-op with either flag value
    for fn in (N.lib.lpmm_b200_adamw4bit_unfused_step_many_flags, N.lib.lpmm_b200_adamw4bit_fused_arith_step_many_flags):
        assert fn(None, 0, qm, qm, 0.9, 0.999, 1e-3, 0.01, 1e-8, None, None, 0, None, 2) == -3
        assert fn(None, 0, qm, qm, 0.9, 0.999, 1e-3, 0.01, 1e-8, None, None, 0, None, 1) == 0
        assert fn(None, 0, qm, qm, 0.9, 0.999, 1e-3, 0.01, 1e-8, None, None, 0, None, 0) == 0


def test_reference_arm_of_the_bench_prints_its_line(tmp_path):
    """``bench.py --impl reference`` on the host cores: one JSON line with the keys of the contract; the reference's own
    Python when ``oracle/_ref/lpmm_py`` (or a checkout) is there, else the C port."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0",
                          "--no-port"], capture_output=True, text=True, timeout=600, cwd=str(tmp_path))
    assert res.returncode == 0, res.stderr[-1000:]
    line = [ln for ln in res.stdout.splitlines() if ln.startswith("{")][-1]
    d = json.loads(line)
    assert d["impl"] == "reference" and d["metric"] == "optimizer_params_updated_per_second" and d["unit"] == "params/s"
    assert d["cpu_baseline"]["kind"] in ("reference-python", "port") and d["cpu_baseline"]["cores"] >= 1
    assert d["value"] > 0 and d["e2e"]["value"] == d["value"] and d["e2e"]["h2d_bytes_per_step"] == 0
    from oracle import build_ref
    if build_ref.have_python() or build_ref.reference_root() is not None:
        assert d["cpu_baseline"]["kind"] == "reference-python"


def test_step_from_host_checks_its_arguments_before_touching_a_gpu():
    """``AdamW.step_from_host``: one entry per parameter, sizes and dtypes checked; an all-``None`` list is a no-op."""
    import torch
    import lpmm
    ps = [torch.nn.Parameter(torch.zeros(8, 4)), torch.nn.Parameter(torch.zeros(5))]
    opt = lpmm.optim.AdamW(ps, fused=True)
    with pytest.raises(ValueError):
        opt.step_from_host([None])
    with pytest.raises(RuntimeError):
        opt.step_from_host([torch.zeros(31), None])
    with pytest.raises(RuntimeError):
        opt.step_from_host([torch.zeros(32, dtype=torch.float64), None])
    ps[0].grad = torch.ones(8, 4)
    opt.step_from_host([None, None])          # nobody steps; a skipped parameter loses its gradient
    assert ps[0].grad is None and len(opt.state) == 0
