"""CPU-side checks of the boundary: the library loads, exports every symbol the public header
declares, the ctypes structs match the C structs' sizes, and host-side validation rejects bad calls
before anything is launched (no GPU needed)."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

REPO = Path(__file__).resolve().parent.parent
HEADER = (REPO / "include" / "fla_b200.h").read_text()


def declared_symbols():
    return sorted(set(re.findall(r"FLA_API\s+int\s+(fla_b200_\w+)\s*\(", HEADER)))


def test_header_declares_entry_points():
    syms = declared_symbols()
    for must in ("fla_b200_gdn_chunk_fwd", "fla_b200_gdn_chunk_bwd", "fla_b200_recurrent_gdn", "fla_b200_causal_conv1d_fwd",
                 "fla_b200_causal_conv1d_update", "fla_b200_version"):
        assert must in syms


def test_library_exports_every_declared_symbol(lib):
    for s in declared_symbols():
        assert hasattr(lib, s), f"libfla_b200.so does not export {s}"
    assert lib.fla_b200_version() >= 100


def test_tensor_desc_layout_matches_header():
    from fla_b200._runtime import TensorDesc, FLA_MAX_DIMS
    assert f"#define FLA_MAX_DIMS {FLA_MAX_DIMS}" in HEADER
    assert ctypes.sizeof(TensorDesc) == 8 + 4 + 4 + 8 * FLA_MAX_DIMS * 2
    assert TensorDesc.shape.offset == 16 and TensorDesc.stride.offset == 16 + 8 * FLA_MAX_DIMS


def _c_struct_fields(name):
    m = re.search(r"typedef struct %s \{(.*?)\} %s;" % (name, name), HEADER, re.S)
    assert m, name
    body = re.sub(r"/\*.*?\*/", "", m.group(1), flags=re.S)
    fields = []
    for decl in body.split(";"):
        decl = decl.strip()
        if not decl:
            continue
        ctype, names = decl.split(None, 1)
        fields += [(ctype, n.strip()) for n in names.split(",")]
    return fields


@pytest.mark.parametrize("cname,pyname", [("fla_recurrent_gdn_args", "RecurrentGdnArgs"),
                                          ("fla_causal_conv1d_fwd_args", "CausalConv1dFwdArgs"),
                                          ("fla_causal_conv1d_update_args", "CausalConv1dUpdateArgs"),
                                          ("fla_causal_conv1d_bwd_args", "CausalConv1dBwdArgs"),
                                          ("fla_gdn_chunk_fwd_args", "GdnChunkFwdArgs"),
                                          ("fla_gdn_chunk_bwd_args", "GdnChunkBwdArgs"),
                                          ("fla_kda_chunk_fwd_args", "KdaChunkFwdArgs"),
                                          ("fla_kda_chunk_bwd_args", "KdaChunkBwdArgs"),
                                          ("fla_kda_intermediates_args", "KdaIntermediatesArgs"),
                                          ("fla_kda_gate_args", "KdaGateArgs"),
                                          ("fla_kda_merge_blocks_args", "KdaMergeBlocksArgs"),
                                          ("fla_kda_merge_inter_args", "KdaMergeInterArgs"),
                                          ("fla_l2norm_args", "L2NormArgs"),
                                          ("fla_fast_gelu_args", "FastGeluArgs"),
                                          ("fla_chunk_stage_args", "ChunkStageArgs"),
                                          ("fla_chunk_kda_bwd_intra_args", "ChunkKdaBwdIntraArgs")])
def test_arg_structs_match_header_field_order(cname, pyname):
    from fla_b200.ops import _structs
    from fla_b200._runtime import TensorDesc
    py = getattr(_structs, pyname)._fields_
    c = _c_struct_fields(cname)
    assert [n for _, n in c] == [n for n, _ in py]
    cmap = {"fla_tensor_t": TensorDesc, "float": ctypes.c_float, "int32_t": ctypes.c_int32}
    for (ctype, n), (pn, pt) in zip(c, py):
        assert cmap[ctype] is pt, (n, ctype, pt)


def test_desc_of_none_and_strided_tensor():
    from fla_b200._runtime import desc
    d = desc(None)
    assert not d.data and d.ndim == 0
    t = torch.zeros(2, 6, 4, dtype=torch.bfloat16)[:, ::2]
    d = desc(t)
    assert d.ndim == 3 and list(d.shape[:3]) == [2, 3, 4] and list(d.stride[:3]) == [24, 8, 1] and d.dtype == 1


def test_cpu_tensors_are_rejected_without_fallback():
    from fla_b200.ops import chunk_gated_delta_rule, causal_conv1d
    q = torch.zeros(1, 64, 1, 128, dtype=torch.bfloat16)
    g = torch.zeros(1, 64, 1)
    with pytest.raises(RuntimeError, match="CUDA device"):
        chunk_gated_delta_rule(q, q, q, g, g)
    with pytest.raises(RuntimeError, match="CUDA device"):
        causal_conv1d(torch.zeros(1, 4, 8, dtype=torch.bfloat16), torch.zeros(8, 4, dtype=torch.bfloat16))


def test_null_and_shape_errors_return_status_codes(lib):
    from fla_b200.ops._structs import GdnChunkFwdArgs, RecurrentGdnArgs
    n = ctypes.c_uint64(0)
    assert lib.fla_b200_gdn_chunk_fwd_workspace_size(None, ctypes.byref(n)) == 1
    a = GdnChunkFwdArgs()
    assert lib.fla_b200_gdn_chunk_fwd(ctypes.byref(a), None, 0, None) == 5          # workspace missing
    buf = ctypes.create_string_buffer(256)
    assert lib.fla_b200_gdn_chunk_fwd(ctypes.byref(a), buf, 256, None) == 1          # null tensors
    r = RecurrentGdnArgs()
    assert lib.fla_b200_recurrent_gdn(ctypes.byref(r), None, 0, None) == 1
    assert lib.fla_b200_selftest_mma(None, None, None, 128, 64, 64, 0, 0, 0, 0, None, None) == 1


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    import fla_b200
    monkeypatch.setattr(fla_b200, "_LIB", None)
    monkeypatch.setenv("FLA_B200_LIB", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no fallback"):
        fla_b200.load_library()
    monkeypatch.delenv("FLA_B200_LIB")
    monkeypatch.setattr(fla_b200, "_LIB", None)
    fla_b200.load_library()
