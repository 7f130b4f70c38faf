"""CPU-side checks of the C-ABI library: it builds, loads, exports every symbol the public header
declares, and validates arguments without needing a GPU (no compute call is made here)."""
import ctypes
import os
import re

import pytest

from dtb200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "dtb200_attn.h")


def _declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dtb_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    declared = _declared_functions()
    assert declared, "no declarations found in the header"
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/dtb200_attn.h but not exported"
    assert sorted(_lib.EXPORTED_SYMBOLS) == declared


def test_struct_layout_matches_header():
    # 4 pointers, 6 int32, 12 int64, 2 pointers, float, uint32, int32, (pad), pointer
    assert ctypes.sizeof(_lib.AttnParams) == 4 * 8 + 6 * 4 + 12 * 8 + 2 * 8 + 4 + 4 + 4 + 4 + 8
    assert ctypes.sizeof(_lib.AttnResidual) == 3 * 8 + 3 * 4 + 4


def _params(**kw):
    p = _lib.AttnParams()
    p.q = p.k = p.v = p.o = 4096
    p.B, p.Hq, p.Hkv, p.Sq, p.Skv, p.D = 1, 4, 4, 512, 512, 128
    p.q_stride_s = p.k_stride_s = p.v_stride_s = p.o_stride_s = 128
    p.q_stride_h = p.k_stride_h = p.v_stride_h = p.o_stride_h = 512 * 128
    p.q_stride_b = p.k_stride_b = p.v_stride_b = p.o_stride_b = 4 * 512 * 128
    for k, v in kw.items():
        setattr(p, k, v)
    return p


@pytest.mark.parametrize("kw,code", [
    ({"D": 64}, 3),                 # head_dim other than 128
    ({"Hkv": 3}, 3),                # query heads not a multiple of kv heads
    ({"Sq": 0}, 3),
    ({"q": None}, 1),
    ({"o": 4100}, 4),               # output pointer not 16-byte aligned
    ({"o_stride_s": 132}, 4),       # output row stride not a multiple of 16 bytes
    ({"flags": _lib.FLAG_BOUNDED_LOGITS}, 1),   # bounded-logit mode without its operand
])
def test_argument_validation_without_a_device(kw, code):
    lib = _lib.load()
    why = ctypes.c_int(-1)
    assert lib.dtb_attn_supported(ctypes.byref(_params(**kw)), ctypes.byref(why)) == 0
    assert why.value == code
    assert lib.dtb_attn_fwd(ctypes.byref(_params(**kw)), None, 0, None) == code


def test_workspace_query_and_status_strings():
    lib = _lib.load()
    assert lib.dtb_version() >= 100
    assert lib.dtb_attn_workspace_bytes(ctypes.byref(_params())) == 0            # 2 q-blocks x 4 heads, short keys
    p = _params(Sq=128, Skv=8192, num_splits=4)
    assert lib.dtb_attn_workspace_bytes(ctypes.byref(p)) == 4 * 1 * 4 * 128 * (128 + 2) * 4
    p = _params(Sq=128, Skv=8192, num_splits=0, Hq=2, Hkv=2)                      # automatic split for a short-query call
    assert lib.dtb_attn_workspace_bytes(ctypes.byref(p)) > 0
    for code, name in _lib.STATUS_NAMES.items():
        assert _lib.status_string(code)
    assert _lib.status_string(12345) == "unknown status"


def test_status_maps_to_reference_exception_types():
    with pytest.raises(NotImplementedError):
        _lib.check(3, "x")
    with pytest.raises(ValueError):
        _lib.check(4, "x")
    with pytest.raises(RuntimeError):
        _lib.check(7, "x")
    _lib.check(0, "x")


def test_python_api_refuses_cpu_tensors():
    import torch

    import dtb200

    q = torch.zeros(1, 2, 128, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        dtb200.attention(q, q, q)
    with pytest.raises(ValueError, match="use_fixed_m needs"):
        dtb200.residual_attention(q, q, q, use_fixed_m=True)


def test_broadcast_and_misaligned_views_are_rejected_before_any_launch():
    """A stride of zero on an axis longer than one (an expanded K/V) cannot be described to TMA; scratch and
    running-state pointers are accessed 16 bytes at a time.  Both are refused with a status, not a GPU fault."""
    lib = _lib.load()
    assert lib.dtb_attn_fwd(ctypes.byref(_params(k_stride_h=0)), None, 0, None) == 3      # DTB_ERR_SHAPE
    assert lib.dtb_attn_fwd(ctypes.byref(_params(v_stride_s=0)), None, 0, None) == 3
    assert lib.dtb_attn_fwd(ctypes.byref(_params(B=2, q_stride_b=0)), None, 0, None) == 3
    # a size-1 axis may carry any stride
    why = ctypes.c_int(-1)
    lib.dtb_attn_supported(ctypes.byref(_params(Hq=1, Hkv=1, q_stride_h=0, k_stride_h=0, v_stride_h=0)), ctypes.byref(why))
    assert why.value in (0, 5)                                                              # ok, or no sm_100 device here
    # residual state / finalize: o_acc must be 16-byte aligned
    r = _lib.AttnResidual(4104, 4096, 4096, 0, 0, 1)
    assert lib.dtb_attn_fwd_residual(ctypes.byref(_params()), ctypes.byref(r), None) == 4   # DTB_ERR_ALIGN
    assert lib.dtb_attn_finalize(ctypes.byref(_params()), ctypes.byref(r), None) == 4
    # bounded-logit operand pass reads rows 8 bytes per lane
    assert lib.dtb_fixed_m_operands(ctypes.byref(_params(q_stride_s=130)), ctypes.c_float(213.0), 4096, 4096, None) == 4


def test_smooth_k_argument_validation():
    lib = _lib.load()
    assert lib.dtb_smooth_k_scratch_bytes(2, 3) == 64 * 2 * 3 * 128 * 4
    sp = _lib.SmoothKParams()
    assert lib.dtb_smooth_k(ctypes.byref(sp), None) == 1                                    # null pointers
    sp.k = sp.out = sp.scratch = 4096
    sp.B, sp.H, sp.S, sp.D = 1, 2, 256, 128
    sp.k_stride_s = sp.out_stride_s = 128
    sp.k_stride_h = sp.out_stride_h = 256 * 128
    sp.k_stride_b = sp.out_stride_b = 2 * 256 * 128
    sp.scratch_bytes = 16
    assert lib.dtb_smooth_k(ctypes.byref(sp), None) == 6                                    # scratch too small
    sp.scratch_bytes = lib.dtb_smooth_k_scratch_bytes(1, 2)
    sp.k_stride_s = 132
    assert lib.dtb_smooth_k(ctypes.byref(sp), None) == 4                                    # rows not 16-byte aligned
    sp.k_stride_s = 128
    sp.D = 64
    assert lib.dtb_smooth_k(ctypes.byref(sp), None) == 3
    assert lib.dtb_fixed_m_from_norms(None, None, 4, 4, ctypes.c_float(0.0), None, None) == 1
    assert lib.dtb_fixed_m_from_norms(4096, 4096, 4, 3, ctypes.c_float(0.0), 4096, None) == 3


def _shape(B, H, S):
    p = _params(B=B, Hq=H, Hkv=H, Sq=S, Skv=S, num_splits=0)
    p.q_stride_h = p.k_stride_h = p.v_stride_h = p.o_stride_h = S * 128
    p.q_stride_b = p.k_stride_b = p.v_stride_b = p.o_stride_b = H * S * 128
    return p


def test_balanced_launch_is_planned_from_the_static_shape():
    """Automatic mode cuts the last wave of a launch into equal runs of key tiles only where that beats the plain
    launch: the scratch request (one 256-row state per piece) says which shapes those are on a 148-SM part."""
    lib = _lib.load()
    slot = 256 * (128 + 2) * 4
    full_c2 = lib.dtb_attn_workspace_bytes(ctypes.byref(_shape(2, 24, 4608)))          # 864 units: 5.84 waves, runs too long to pay
    quarter_c2 = lib.dtb_attn_workspace_bytes(ctypes.byref(_shape(1, 12, 4608)))       # 216 units: a 68-unit last wave
    eighth_c2 = lib.dtb_attn_workspace_bytes(ctypes.byref(_shape(1, 6, 4608)))         # 108 units of 36 tiles: runs of 27 do not pay
    eighth_c3 = lib.dtb_attn_workspace_bytes(ctypes.byref(_shape(1, 6, 16896)))        # 396 units of 132 tiles
    exact = lib.dtb_attn_workspace_bytes(ctypes.byref(_shape(1, 37, 1024)))            # 148 units: one full wave
    assert full_c2 == 0 and eighth_c2 == 0 and exact == 0
    for need in (quarter_c2, eighth_c3):
        assert need > 0 and need % slot == 0 and need // slot <= 2 * 148
    # forced modes keep their meaning
    assert lib.dtb_attn_workspace_bytes(ctypes.byref(_params(Sq=128, Skv=8192, num_splits=1))) == 0


def test_out_proj_argument_validation():
    lib = _lib.load()
    p = _lib.OutProjParams()
    assert lib.dtb_out_proj(ctypes.byref(p), None) == 1                       # null operands
    p.o = p.w = p.out = 4096
    p.B, p.H_local, p.S, p.D, p.N = 1, 2, 256, 128, 384
    p.o_stride_s, p.o_stride_h, p.o_stride_b = 128, 256 * 128, 2 * 256 * 128
    p.w_stride_k, p.out_stride_s, p.out_stride_b = 384, 384, 256 * 384
    p.N = 100
    assert lib.dtb_out_proj(ctypes.byref(p), None) == 3                       # N not a multiple of 8
    p.N = 384
    p.D = 64
    assert lib.dtb_out_proj(ctypes.byref(p), None) == 3
    p.D = 128
    p.out = 4100
    assert lib.dtb_out_proj(ctypes.byref(p), None) == 4                       # misaligned output
    p.out = 4096
    p.n_dest, p.rows_per_dest = 2, 64                                         # two destinations cannot hold 256 rows
    p.red_dst[0] = p.red_dst[1] = 4096
    assert lib.dtb_out_proj(ctypes.byref(p), None) == 3
    p.rows_per_dest = 128
    p.red_dst[1] = None
    assert lib.dtb_out_proj(ctypes.byref(p), None) == 1
    assert lib.dtb_sum_partials(None, 2, 16, 128, None, None) == 1
    assert lib.dtb_sum_partials(4096, 9, 16, 128, 4096, None) == 3


@pytest.mark.parametrize("B,H,S,sms", [(1, 12, 4608, 148), (1, 6, 16896, 148), (1, 2, 256, 148), (2, 24, 16896, 148),
                                       (1, 12, 4608, 132), (1, 5, 48872, 148), (3, 7, 2000, 100)])
def test_launch_plan_covers_every_key_tile_exactly_once(B, H, S, sms):
    """The work list of a balanced launch: whole units first, then pieces that tile the key range of every unit of
    the last wave exactly once, longest first, with consecutive scratch slots per unit in key order."""
    lib = _lib.load()
    p = _shape(B, H, S)
    if (B, H, S) == (1, 2, 256, 148):
        p = _shape(1, 2, 256)
        p.Skv = 8192
    plan = _lib.LaunchPlan()
    assert lib.dtb_attn_launch_plan(ctypes.byref(p), sms, ctypes.byref(plan)) == 0
    n = plan.key_tiles
    assert plan.units == B * H * ((p.Sq + 255) // 256) and plan.tail_units == plan.units % sms
    if plan.n_pieces == 0:
        assert plan.whole_units == plan.units and plan.n_slots == 0
        return
    assert plan.whole_units == plan.units - plan.tail_units and plan.whole_units % sms == 0
    pieces = [(plan.unit[i], plan.tile_begin[i], plan.tile_end[i], plan.slot[i]) for i in range(plan.n_pieces)]
    lens = [te - tb for _, tb, te, _ in pieces]
    assert lens == sorted(lens, reverse=True) and min(lens) >= 1
    by_unit = {}
    for u, tb, te, slot in pieces:
        assert plan.whole_units <= u < plan.units
        by_unit.setdefault(u, []).append((tb, te, slot))
    assert len(by_unit) == plan.tail_units
    slots_seen = []
    for u, ps in by_unit.items():
        ps.sort()
        assert ps[0][0] == 0 and ps[-1][1] == n
        for (a0, a1, _), (b0, b1, _) in zip(ps, ps[1:]):
            assert a1 == b0                                   # no gap, no overlap
        if len(ps) == 1:
            assert ps[0][2] == -1                             # swept whole: writes the output itself
        else:
            s = [x[2] for x in ps]
            assert s == list(range(s[0], s[0] + len(s)))      # consecutive slots in key order
            slots_seen += s
    assert sorted(slots_seen) == list(range(plan.n_slots))
    # every SM's share: the runs are equal to within one tile
    assert max(lens) <= -(-plan.tail_units * n // min(sms, plan.tail_units * n // 4)) 
    assert lib.dtb_attn_workspace_bytes(ctypes.byref(p)) in (0, plan.n_slots * 256 * 130 * 4) or sms != 148


def test_describe_launch_names_the_form():
    import dtb200

    assert "plain launch" in dtb200.describe_launch(2, 24, 4608)
    assert "cut into" in dtb200.describe_launch(1, 12, 4608)
