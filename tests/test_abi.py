"""CPU: the C-ABI library loads and exports every symbol include/mok_b200.h declares; argument
errors the host can detect come back as codes without touching a GPU."""
import ctypes
import os
import re

from tests.conftest import ROOT


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "mok_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mok_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported():
    import mok
    names = _declared_symbols()
    assert len(names) >= 12
    for n in names:
        assert hasattr(mok._lib.lib, n), f"{n} declared in mok_b200.h but not exported"


def test_version_and_error_strings():
    import mok
    assert mok._lib.mok_version() >= 100
    assert mok._lib.mok_error_string(-1) == b"invalid argument"
    assert mok._lib.mok_error_string(1) == b"schedule capacity exceeded"


def test_host_detected_argument_errors():
    import mok
    L = mok._lib
    assert L.mok_schedule_scratch_bytes(8, 32) == (8 * 256 * 32 + 8 * 32) * 4
    assert L.mok_schedule(None, 4, 512, 2, 4, 4096, 0, None, None, None, None, None, 0, None, None) == -1
    assert L.mok_mxfp8_quantize(None, 1, 128, 128, None, None, None, None, None) == -1
    assert L.mok_gemm_bf16(ctypes.c_void_p(16), ctypes.c_void_p(16), ctypes.c_void_p(16), 100, 256, 64, 0, 0, None, None) == -1
    assert L.mok_fwd_bf16(None, None) == -1
    assert L.mok_barrier_all(None, None, 4, None, None, 0, None) == -1
    # entry points without a reference counterpart
    p16 = ctypes.c_void_p(16)
    assert L.mok_router_topk(None, 512, 64, 6, None, None, None, None, 0, 0, None) == -1
    assert L.mok_router_topk(p16, 512, 64, 65, p16, None, p16, None, 0, 0, None) == -1          # topk > 32
    assert L.mok_router_topk(p16, 512, 2048, 4, p16, None, p16, None, 0, 0, None) == -3         # more than 1024 experts
    assert L.mok_router_topk_bwd(None, None, None, None, 512, 64, 6, None) == -1
    assert L.mok_fwd_epilogue_rows(None, None, None, None, None, None, None, None, 512, 256, 2, 4096, None) == -1
    assert L.mok_bwd_epilogue_rows(None, None, None, 4, None, None, None, None, None, None, 512, 256, 2, 4096, None) == -1
    assert L.mok_last_cuda_error() == b""
    assert L.mok_last_status(None, None, 0, None) == -1


def test_query_workspace_bytes():
    """The size query follows the reference's capacity formula T*K*max(2, ceil(W*multiplier)) and buffer shapes."""
    import mok
    L = mok._lib
    wb = L.WorkspaceBytes()
    assert L.mok_query_workspace_bytes(8, 16384, 7168, 8, 32, 0.5, wb) == 0
    R = 16384 * 8
    assert wb.schedule_capacity == R * 4
    assert wb.x_buffer == wb.d_y_buffer == 16384 * 7168 * 2
    assert wb.combine_buffer == wb.d_x_routed_buffer == R * 7168 * 2
    assert wb.router_weight_buffer == wb.d_router_weight_buffer == R * 4
    assert wb.all_gather_top_experts_buffer == 8 * R * 4
    assert (wb.barrier_buffer, wb.barrier_target, wb.status_word) == (4, 4, 16)
    assert wb.schedule_tables == 2 * 4 * R * 4 + 4 + 32 * 4
    assert wb.schedule_scratch == L.mok_schedule_scratch_bytes(8, 32)
    assert L.mok_query_workspace_bytes(1, 512, 256, 2, 4, 1.0, wb) == 0 and wb.schedule_capacity == 512 * 2 * 2
    assert L.mok_query_workspace_bytes(8, 16384, 7168, 8, 32, 1.0, wb) == 0 and wb.schedule_capacity == R * 8
    for bad in ((0, 512, 256, 2, 4, 1.0), (9, 512, 256, 2, 4, 1.0), (1, 500, 256, 2, 4, 1.0), (1, 512, 100, 2, 4, 1.0),
                (1, 512, 256, 0, 4, 1.0), (1, 512, 256, 2, 0, 1.0), (1, 512, 256, 2, 4, 0.0)):
        assert L.mok_query_workspace_bytes(*bad, wb) == -1, bad
    assert L.mok_query_workspace_bytes(1, 512, 256, 2, 4, 1.0, None) == -1


def test_struct_sizes_match_header():
    """The ctypes mirrors must have the same size as the C structs (checked with gcc)."""
    import subprocess
    import tempfile
    import mok
    src = '#include <stdio.h>\n#include "mok_b200.h"\nint main(){printf("%zu %zu %zu %zu %zu %zu", sizeof(mok_layer_common), sizeof(mok_fwd_bf16_args), sizeof(mok_bwd_bf16_args), sizeof(mok_fwd_mxfp8_args), sizeof(mok_bwd_mxfp8_args), sizeof(mok_workspace_bytes));return 0;}\n'
    with tempfile.TemporaryDirectory() as d:
        c = os.path.join(d, "s.c")
        open(c, "w").write(src)
        exe = os.path.join(d, "s")
        subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), c, "-o", exe])
        sizes = [int(v) for v in subprocess.check_output([exe]).split()]
    L = mok._lib
    assert sizes == [ctypes.sizeof(L.LayerCommon), ctypes.sizeof(L.FwdBf16Args), ctypes.sizeof(L.BwdBf16Args),
                     ctypes.sizeof(L.FwdMxfp8Args), ctypes.sizeof(L.BwdMxfp8Args), ctypes.sizeof(L.WorkspaceBytes)]


def test_ctypes_field_order_matches_header():
    """Same sizes are not enough: every struct member must sit where the header puts it."""
    import mok
    L = mok._lib
    text = re.sub(r"/\*.*?\*/", "", open(os.path.join(ROOT, "include", "mok_b200.h")).read(), flags=re.S)
    pairs = (("mok_layer_common", L.LayerCommon), ("mok_fwd_bf16_args", L.FwdBf16Args),
             ("mok_bwd_bf16_args", L.BwdBf16Args), ("mok_fwd_mxfp8_args", L.FwdMxfp8Args),
             ("mok_bwd_mxfp8_args", L.BwdMxfp8Args), ("mok_workspace_bytes", L.WorkspaceBytes))
    type_words = {"const", "void", "uint64_t", "int32_t", "int64_t", "size_t", "int", "float", "mok_layer_common"}
    for cname, struct in pairs:
        body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (cname, cname), text, re.S).group(1)
        names = [w for decl in body.split(";") for w in decl.replace("*", " ").replace(",", " ").split()
                 if w not in type_words]
        assert names == [f[0] for f in struct._fields_], cname
