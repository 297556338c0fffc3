"""Host-side logic on CPU: packers against the oracle and the golden vectors, the
C-ABI library's exports, and argument validation (no compute without a GPU)."""
import ctypes
import re
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import formats, int4, nvfp4
from turbopi_b200 import _lib, nvfp4_packed, w4a16

ROOT = Path(__file__).resolve().parent.parent


def test_library_exports_every_declared_symbol():
    header = (ROOT / "include" / "turbopi_b200.h").read_text()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(tpb200_\w+|nvfp4_gemv_\w+|quantize\w+|dequantize\w+|w4a16Gemm\w+|w4a8Gemm\w+|"
                              r"getW4A\w+)\s*\(", header))
    declared -= {"tpb200_status", "tpb200_stream_t", "tpb200_gemv_problem"}
    assert declared, "no declarations found"
    lib = ctypes.CDLL(str(_lib.LIB_PATH))
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} declared in include/turbopi_b200.h but not exported"
    assert declared == set(_lib.SIGNATURES), (declared ^ set(_lib.SIGNATURES))
    assert _lib.load().tpb200_version() >= 100


def test_argument_validation_happens_on_the_host():
    lib = _lib.load()
    # NULL pointers, bad shapes, bad enums: rejected before any CUDA call
    assert lib.tpb200_nvfp4_gemv(None, 2, None, None, None, 1, 16, 1.0, None, 0, None, 2, 1, 64, 64, 0, 0, None) == -1
    assert lib.tpb200_nvfp4_gemv(16, 2, None, 16, 16, 1, 16, 1.0, None, 0, 16, 2, 17, 64, 64, 0, 0, None) == -2
    assert lib.tpb200_nvfp4_gemv(16, 2, None, 16, 16, 1, 16, 1.0, None, 0, 16, 2, 1, 64, 48, 0, 0, None) == -2
    assert lib.tpb200_nvfp4_gemv(16, 7, None, 16, 16, 1, 16, 1.0, None, 0, 16, 2, 1, 64, 64, 0, 0, None) == -4
    assert lib.tpb200_nvfp4_gemv(16, 2, None, 8, 16, 1, 16, 1.0, None, 0, 16, 2, 1, 64, 64, 0, 0, None) == -3
    assert lib.tpb200_w4a16_gemv(16, 1, 16, 16, 2, None, 0, 16, 0, 1, 64, 64, 32, 9, 0, None) == -4
    assert lib.tpb200_w4a16_gemv(16, 1, 16, 16, 2, None, 0, 16, 0, 1, 64, 64, 64, 0, 0, None) == -2
    lib.quantizeWeightToINT4(None, None, None, None, 4, 128, 128, None)
    assert lib.tpb200_last_error() == -1 and lib.tpb200_last_error() == 0
    assert b"NULL" in lib.tpb200_status_string(-1)


def test_ops_refuse_cpu_tensors():
    from turbopi_b200 import ops
    x = torch.zeros(1, 64, dtype=torch.float16)
    with pytest.raises(_lib.TurboPiError):
        ops.w4a16_gemv(x, torch.zeros(2, 8, 4, dtype=torch.int32), torch.zeros(2, 8, dtype=torch.float16))
    with pytest.raises(_lib.TurboPiError):
        ops.nvfp4_gemv_v6(torch.zeros(1, 64), torch.zeros(8, 32, dtype=torch.uint8), torch.zeros(8, 2), None, 1, 8, 64, 0)


def test_int4_packers_match_oracle_and_golden(golden):
    g = golden("int4_packers")
    w = torch.from_numpy(g["weight"])
    fast = w4a16.W4A16PackerFast().pack(w)
    assert fast.weight_packed.dtype == torch.int32 and fast.scales.dtype == torch.float16
    assert np.array_equal(fast.weight_packed.numpy(), g["fast_packed"].astype(np.int32))
    assert np.array_equal(fast.scales.numpy().view(np.uint16), g["fast_scales"].view(np.uint16))
    basic = w4a16.W4A16Packer().pack(w)
    assert np.array_equal(basic.weight_packed.numpy(), g["basic_packed"])
    assert np.array_equal(basic.scales.numpy().view(np.uint16), g["basic_scales"].view(np.uint16))
    assert np.array_equal(w4a16.W4A16Packer().unpack(basic).numpy(), g["basic_unpacked"])
    words, scales = w4a16.W4A16PackerFast().pack_rowmajor(w, 128)
    ow, os_ = int4.pack_fast(g["weight"], 128, "rowmajor")
    assert np.array_equal(words.numpy(), ow) and np.array_equal(scales.numpy().view(np.uint16), os_.view(np.uint16))


def test_int4_state_dict_roundtrip_and_autopack():
    torch.manual_seed(0)
    lin = torch.nn.Linear(64, 24, bias=True)
    q = w4a16.W4A16Linear.from_linear(lin)
    sd = q.state_dict()
    assert set(sd) == {"weight_packed", "scales", "bias"}
    q2 = w4a16.W4A16Linear(64, 24, bias=True)
    q2.load_state_dict(sd)
    assert torch.equal(q2.weight_packed, q.weight_packed) and torch.equal(q2.scales, q.scales)
    q3 = w4a16.W4A16Linear(64, 24, bias=True)
    q3.load_state_dict({"weight": lin.weight.data, "bias": lin.bias.data})      # unpacked weight: quantised on load
    assert torch.equal(q3.weight_packed, q.weight_packed)
    assert q.weight.dtype == torch.float16 and q.weight.shape == (24, 64)
    assert (q.weight.float() - lin.weight).abs().max() < lin.weight.abs().max() / 7


def test_nvfp4_packers_match_oracle_and_golden(golden):
    g = golden("nvfp4_packed")
    w = torch.from_numpy(g["weight"])
    q, s = nvfp4_packed.quantize_to_nvfp4(w, 32)
    assert np.array_equal(q.numpy(), g["quantized"]) and np.array_equal(s.numpy(), g["scales"])
    p = nvfp4_packed.pack_nvfp4(q)
    assert np.array_equal(p.numpy(), g["packed"])
    assert np.array_equal(nvfp4_packed.unpack_nvfp4(p, 40, 128).numpy(), g["unpacked"])
    rng = np.random.default_rng(5)
    w2 = (rng.normal(size=(32, 256)) * 0.02).astype(np.float32)
    w2[3, :16] = 0
    pk, sc, gs = nvfp4_packed.quantize_nvfp4_two_level(torch.from_numpy(w2), 16)
    opk, osc, ogs = nvfp4.quantize_two_level(w2, 16)
    assert gs == float(ogs)
    assert np.array_equal(sc.numpy(), osc)
    assert np.array_equal(pk.numpy(), opk)
    deq = nvfp4.dequantize(opk, osc, 16, ogs, scale_is_e4m3=True)
    assert np.abs(deq - w2).max() < np.abs(w2).max() * 0.3


def test_nvfp4_sim_quantiser_matches_golden(golden):
    from turbopi_b200 import nvfp4_linear
    g = golden("nvfp4_sim")
    w = torch.from_numpy(g["weight"])
    q, s = nvfp4_linear.quantize_to_nvfp4_sim(w, 32, use_mse_search=True)
    assert np.array_equal(q.numpy(), g["wq_mse"]) and np.array_equal(s.numpy(), g["ws_mse"])
    q2, s2 = nvfp4_linear.quantize_to_nvfp4_sim(w, 32, use_mse_search=False)
    assert np.array_equal(q2.numpy(), g["wq_minmax"]) and np.array_equal(s2.numpy(), g["ws_minmax"])
    d = nvfp4_linear.dequantize_nvfp4_sim(q, s, 32, use_fp8_scales=True)
    assert np.array_equal(d.numpy(), g["w_dequant_fp8"])
    assert np.array_equal(nvfp4_linear.pack_nvfp4_data(q).numpy(), g["w_packed"])
    sw = nvfp4_linear.prepare_scales(s, 32).numpy()
    ref = nvfp4.swizzle_scales_128x4(np.repeat(formats.e4m3_encode(g["ws_mse"]), 2, axis=1), 16)
    assert np.array_equal(sw, ref)


def test_weight_row_permutations_are_permutations():
    """The fused-QKV and gated-GELU epilogues rely on the weight rows being re-ordered; both orders must be
    permutations with the documented block structure."""
    import torch
    from turbopi_b200 import ops
    p = ops.qkv_tile_permutation(2048)
    assert sorted(p.tolist()) == list(range(2048 + 512))
    t = p.reshape(-1, 128)                               # every 128-row tile: 64 rows, then the same + 128
    assert (t[:, 64:] == t[:, :64] + 128).all()
    g = ops.geglu_row_permutation(1024)
    assert sorted(g.tolist()) == list(range(2048))
    b = g.reshape(-1, 2, 128)                            # every 256-row block: 128 gate rows, their up rows
    assert (b[:, 1] == b[:, 0] + 1024).all() and (b[:, 0, 0] == torch.arange(8) * 128).all()


def _gemv_tc_plan(shapes, sms=148):
    n = len(shapes)
    N = (ctypes.c_int * n)(*[s[0] for s in shapes])
    K = (ctypes.c_int * n)(*[s[1] for s in shapes])
    info = _lib.GemvTcPlanInfo()
    status = _lib.load().tpb200_nvfp4_gemv_tc_plan(N, K, n, sms, ctypes.byref(info))
    return status, info


def test_gemv_tc_planner_covers_every_stage_and_fits_the_gpu():
    """The tensor-core GEMV's launch planner runs on the host alone: every 256-row x 256-column stage of every
    matrix is planned exactly once, the grid never exceeds the SM count, and scratch is asked for only when tiles
    are cut along K or units are pooled."""
    stages = lambda shapes: sum(-(-n // 256) * (k // 256) for n, k in shapes)
    expert = [(4096, 1024), (4096, 1024), (1024, 4096)] * 18          # the 54 MLP matrices of the action expert
    status, info = _gemv_tc_plan(expert)
    assert status == 0
    assert info.grid == 148 and info.total_stages == stages(expert) == 3456
    assert info.pool_units > 0 and info.pool_units + info.grid == info.units    # one fixed unit per CTA, rest pooled
    assert info.max_load_stages * info.grid < info.total_stages                  # the pool carries most of the work
    assert info.workspace_bytes >= 4                                             # the pool's ticket counter

    for shapes in ([(4096, 1024)], [(16384, 2048)], [(256, 256)], [(100, 256)]):
        status, info = _gemv_tc_plan(shapes)
        assert status == 0 and info.total_stages == stages(shapes)
        assert 1 <= info.grid <= 148 and info.cut_tiles == 0 and info.workspace_bytes == 0

    status, info = _gemv_tc_plan([(1024, 4096)])          # 4 row tiles of 16 stages: cut along K to fill more SMs
    assert status == 0 and info.cut_tiles == 4 and info.grid > 4 and info.workspace_bytes > 0
    assert info.total_stages == 64

    status, info = _gemv_tc_plan([(4096, 1024)] * 3, sms=8)
    assert status == 0 and info.grid == 8 and info.total_stages == 192

    for bad in ([(4096, 1000)], [(0, 1024)], []):          # K not a multiple of the stage, empty problems
        status, _ = _gemv_tc_plan(bad) if bad else (_lib.load().tpb200_nvfp4_gemv_tc_plan(None, None, 0, 148, None), None)
        assert status != 0


def test_attention_arguments_are_validated_on_the_host():
    """tpb200_attention refuses bad shapes / strides / hand-over requests before any CUDA call (fake 16-byte
    aligned pointers, no device needed)."""
    lib = _lib.load()
    two = ctypes.c_longlong * 2

    def args(**kw):
        a = dict(q=256, k=256, v=256, out=256, key_bias=None, n_rows=64, n_keys=300, head_dim=256, ldq=256, ldk=256,
                 ldv=256, ldo=256, groups_outer=1, groups_inner=1, q_stride=two(0, 0), k_stride=two(0, 0),
                 v_stride=two(0, 0), o_stride=two(0, 0), scale=1.0, workspace=None, workspace_bytes=0, flags=0,
                 quant_image=None, quant_row_scale=None, quant_pieces=0, quant_rows_per_token=1)
        a.update(kw)
        return _lib.AttentionArgs(**a)

    call = lambda **kw: lib.tpb200_attention(ctypes.byref(args(**kw)), None)
    assert call(q=None) == -1
    assert call(head_dim=264) == -2 and call(head_dim=12) == -2 and call(n_keys=0) == -2
    assert call(ldq=128) == -2                         # row stride shorter than a row
    assert call(q=264) == -3 and call(ldk=260) == -3    # not 16-byte aligned
    assert call(flags=8) == -4
    assert call() == -6                                 # two key tiles need the workspace
    # fused hand-over to the next linear: one problem only, whole tokens, K a multiple of 256, 1..3 pieces
    q = dict(quant_image=256, quant_row_scale=256, quant_pieces=3, quant_rows_per_token=8, workspace=256,
             workspace_bytes=1 << 30)
    assert call(**{**q, "groups_inner": 2}) == -2
    assert call(**{**q, "quant_row_scale": None}) == -1
    assert call(**{**q, "quant_pieces": 4}) == -2
    assert call(**{**q, "n_rows": 60}) == -2            # 60 rows are not whole tokens of 8
    assert call(**{**q, "quant_rows_per_token": 2, "head_dim": 72, "ldq": 72, "ldk": 72, "ldv": 72, "ldo": 72}) == -2
    assert lib.tpb200_attention_workspace_size(400, 762, 256, 1) >= 4 * 6 * 128 * (256 + 2) * 4
    assert lib.tpb200_attention_workspace_size(64, 300, 300, 1) == 0


def test_bench_reference_arm_prints_the_contract_line():
    """`bench.py --impl reference` needs no GPU: one JSON line with the own arm's metric, unit and config, the CPU
    baseline it timed (`kind`, `cores`, `sample`) and an `e2e` that repeats the value with no copies."""
    import json
    import subprocess
    import sys
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, timeout=600, cwd=str(ROOT))
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "nvfp4_gemv_hbm_gbps" and d["unit"] == "GB/s"
    assert d["higher_is_better"] is True and d["n_gpus"] == 1 and d["value"] > 0
    assert d["cpu_baseline"]["kind"] in ("port", "reference") and d["cpu_baseline"]["cores"] >= 1
    assert d["cpu_baseline"]["value"] == d["value"] and d["cpu_baseline"]["sample"]
    assert d["e2e"] == {"value": d["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "workload" in d["config"]


def test_ctypes_structures_follow_the_header_field_by_field():
    """Every argument struct of include/turbopi_b200.h has a ctypes mirror in turbopi_b200/_lib.py with the same
    fields in the same order (a field added on one side only would shift everything behind it)."""
    header = (ROOT / "include" / "turbopi_b200.h").read_text()
    mirrors = {"tpb200_gemv_problem": _lib.GemvProblem, "tpb200_nvfp4_gemm_args": _lib.GemmArgs,
               "tpb200_gemv_tc_problem": _lib.GemvTcProblem, "tpb200_gemv_tc_fused_problem": _lib.GemvTcFusedProblem,
               "tpb200_gemv_tc_plan_info": _lib.GemvTcPlanInfo, "tpb200_attention_args": _lib.AttentionArgs,
               "tpb200_rowop_args": _lib.RowOpArgs}
    for name, mirror in mirrors.items():
        m = re.search(r"typedef struct(?:\s+\w+)?\s*\{([^}]*)\}\s*" + name + r"\s*;", header, re.S)
        assert m, name
        body = re.sub(r"/\*.*?\*/", "", m.group(1), flags=re.S)
        fields = [part.strip().split()[-1].split("[")[0].lstrip("*")          # "int M, N, K" declares three
                  for d in body.split(";") if d.strip() for part in d.split(",")]
        assert fields == [f[0] for f in mirror._fields_], name
