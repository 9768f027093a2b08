"""The C-ABI library loads without a GPU and exports every function the header declares; argument
checks that need no device are exercised through ctypes."""
import ctypes as C
import re
from pathlib import Path

import pytest

from sageattention_b200 import _lib

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "sage3_b200.h"


def declared_functions():
    text = HEADER.read_text()
    return re.findall(r"SAGE3_API\s+[\w\s\*]+?\b(sage3_\w+)\s*\(", text)


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = declared_functions()
    assert len(names) >= 8
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/sage3_b200.h but not exported"
    assert set(names) >= set(_lib.EXPORTS)


def test_ctypes_mirrors_have_the_layout_of_the_c_structs(tmp_path):
    """The Python front end fills ctypes mirrors of the header's structs: sizes and the offset of the last field must
    be what a C compiler makes of the header (a field added on one side only would shift everything behind it)."""
    import subprocess
    pairs = {"sage3_shape": _lib.Shape, "sage3_tensor": _lib.Tensor, "sage3_sizes": _lib.Sizes,
             "sage3_quant_args": _lib.QuantArgs, "sage3_attn_args": _lib.AttnArgs, "sage3_fwd_args": _lib.FwdArgs,
             "sage3_pack_args": _lib.PackArgs, "sage3_varlen_args": _lib.VarlenArgs}
    lines = "".join(f'  printf("{n} %zu %zu\\n", sizeof({n}), offsetof({n}, {cls._fields_[-1][0]}));\n'
                    for n, cls in pairs.items())
    src = tmp_path / "layout.c"
    src.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "sage3_b200.h"\nint main(void) {\n' + lines +
                   "  return 0;\n}\n")
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-I", str(HEADER.parent), str(src), "-o", str(exe)], check=True)
    got = {}
    for line in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.splitlines():
        name, size, last = line.split()
        got[name] = (int(size), int(last))
    for n, cls in pairs.items():
        assert got[n] == (C.sizeof(cls), getattr(cls, cls._fields_[-1][0]).offset), n


def test_version_and_status_strings():
    lib = _lib.load()
    assert lib.sage3_version() >= 100
    assert lib.sage3_status_string(0) == b"ok"
    for code in (1, 2, 3, 4):
        assert len(lib.sage3_status_string(code)) > 5
    assert lib.sage3_status_string(99) == b"unknown status"


def test_buffer_sizes_and_shape_checks():
    lib = _lib.load()
    z = _lib.Sizes()
    s = _lib.Shape(1, 8, 8, 1024, 1024, 128)
    assert lib.sage3_buffer_sizes(C.byref(s), 1, C.byref(z)) == _lib.OK
    assert z.q_codes == 8 * 1024 * 64 and z.q_sf == 8 * 8 * 2 * 512
    assert z.vt_codes == 8 * 8 * 128 * 64 and z.vt_sf == 8 * 8 * 1024
    assert z.delta_s == 8 * 8 * 1024 * 2 and z.km == 8 * 128 * 2
    assert z.workspace >= z.q_codes + z.k_codes + z.vt_codes + z.delta_s
    # ragged lengths round up to whole 128-token tiles
    s2 = _lib.Shape(2, 4, 2, 130, 1, 64)
    assert lib.sage3_buffer_sizes(C.byref(s2), 1, C.byref(z)) == _lib.OK
    assert z.q_codes == 2 * 4 * 2 * 128 * 32 and z.k_codes == 2 * 2 * 1 * 128 * 32
    for bad in (_lib.Shape(1, 8, 8, 128, 128, 96), _lib.Shape(1, 3, 2, 128, 128, 128)):
        assert lib.sage3_buffer_sizes(C.byref(bad), 1, C.byref(z)) == _lib.ERR_UNSUPPORTED
    assert lib.sage3_buffer_sizes(C.byref(_lib.Shape(0, 1, 1, 1, 1, 128)), 1, C.byref(z)) == _lib.ERR_ARGUMENT
    assert lib.sage3_buffer_sizes(None, 1, C.byref(z)) == _lib.ERR_ARGUMENT


def test_null_and_misaligned_arguments_are_rejected_before_any_launch():
    lib = _lib.load()
    assert lib.sage3_quant_qkv(None, None) == _lib.ERR_ARGUMENT
    assert lib.sage3_attn_fwd(None, None) == _lib.ERR_ARGUMENT
    assert lib.sage3_attention(None, None) == _lib.ERR_ARGUMENT
    a = _lib.QuantArgs()
    a.shape = _lib.Shape(1, 1, 1, 128, 128, 128)
    a.q = _lib.Tensor(0x1008, 128 * 128, 128 * 128, 128)       # not 16-byte aligned
    assert lib.sage3_quant_qkv(C.byref(a), None) == _lib.ERR_ARGUMENT
    a.q = _lib.Tensor(0x1000, 128 * 128, 128 * 128, 130)        # rows not 16-byte aligned
    assert lib.sage3_quant_qkv(C.byref(a), None) == _lib.ERR_ARGUMENT
    a.q = _lib.Tensor(0x1000, 128 * 128, 128 * 128, 128)        # outputs missing
    assert lib.sage3_quant_qkv(C.byref(a), None) == _lib.ERR_ARGUMENT
    t = _lib.AttnArgs()
    t.shape = _lib.Shape(1, 1, 1, 128, 128, 128)
    assert lib.sage3_attn_fwd(C.byref(t), None) == _lib.ERR_ARGUMENT


def test_front_end_refuses_cpu_tensors():
    import torch
    import sageattention_b200 as sa
    q = torch.zeros(1, 1, 128, 128, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        sa.sageattn(q, q, q)


def test_custom_op_fake_needs_no_gpu():
    """The torch.library registration (the reference does this for its INT8 kernels,
    sageattention/sm89_compile.py:5-101): shape propagation through the fake implementation."""
    import torch
    from sageattention_b200 import compile_ops
    q = torch.empty((2, 8, 300, 128), dtype=torch.bfloat16, device="meta")
    k = torch.empty((2, 2, 500, 128), dtype=torch.bfloat16, device="meta")
    out = compile_ops.sageattn_compilable(q, k, k, is_causal=True)
    assert out.shape == q.shape and out.dtype == torch.bfloat16 and out.device.type == "meta"
    out = compile_ops.sageattn_compilable(q.transpose(1, 2), k.transpose(1, 2), k.transpose(1, 2), tensor_layout="NHD",
                                          k_packing=True)
    assert out.shape == (2, 300, 8, 128)


def test_packed_length_helpers_match_reference_formulas():
    """sage3_packed_len = the key-length fix-up of sageattn4/api.py:267-274; sage3_packed_rows = rows of the
    packed tensors (groups of 15 tokens padded, 16 slots each, api.py:124-127,146)."""
    from oracle import sage3
    lib = _lib.load()
    for n in (1, 14, 15, 16, 29, 30, 31, 100, 128, 8192, 32760, 75600):
        q = 15
        want = n // q * (q + 1) if n % q == 0 else n // q * (q + 1) + 1 + n % q
        assert lib.sage3_packed_len(n) == want == sage3.logical_to_packed_len(n)
        assert lib.sage3_packed_rows(n) == 16 * ((n + 14) // 15)
        assert lib.sage3_packed_rows(n) - 14 <= lib.sage3_packed_len(n) <= lib.sage3_packed_rows(n)
    assert lib.sage3_packed_len(0) == 0 and lib.sage3_packed_rows(-3) == 0
    a = _lib.PackArgs()
    assert lib.sage3_pack_kv(C.byref(a), None) == _lib.ERR_ARGUMENT       # null tensors: refused before any CUDA call


def test_varlen_entry_refuses_bad_arguments_without_a_gpu():
    lib = _lib.load()
    a = _lib.VarlenArgs()
    assert lib.sage3_attention_varlen(C.byref(a), None) == _lib.ERR_ARGUMENT      # no workspace / tensors
    assert lib.sage3_attention_varlen(None, None) == _lib.ERR_ARGUMENT
