"""CPU-only checks of the C ABI: the library loads, exports every declared symbol, the ctypes
mirrors match the C structs byte for byte, and argument validation returns the documented codes
(no kernel is launched: validation fails first)."""
import ctypes as C
import os
import re
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "palimpsa_b200.h")


@pytest.fixture(scope="module")
def L():
    from palimpsa_b200 import _lib, build
    build.build()
    _lib.lib()
    return _lib


def test_exports_every_declared_symbol(L):
    src = open(HEADER).read()
    declared = set(re.findall(r"\b(palimpsa_[a-z_0-9]+)\s*\(", src))
    declared -= {"palimpsa_padded_k"} - set(L.SYMBOLS)  # keep only functions
    h = C.CDLL(L.LIB_PATH)
    assert declared, "no declarations found"
    for name in declared:
        assert hasattr(h, name), f"{name} declared in the header but not exported"
    assert set(L.SYMBOLS) == declared


def test_struct_layout_matches_c(L, tmp_path):
    prog = tmp_path / "layout.c"
    fields_p = [f[0] for f in L.Problem._fields_]
    fields_f = [f[0] for f in L.FwdParams._fields_]
    fields_b = [f[0] for f in L.BwdParams._fields_]
    lines = ['#include <stdio.h>', '#include <stddef.h>', f'#include "{HEADER}"', "int main(){"]
    fields_s = [f[0] for f in L.Segments._fields_]
    fields_lp = [f[0] for f in L.LayerPrologue._fields_]
    fields_le = [f[0] for f in L.LayerEpilogue._fields_]
    for st, fl in (("palimpsa_problem", fields_p), ("palimpsa_fwd_params", fields_f), ("palimpsa_bwd_params", fields_b),
                   ("palimpsa_segments", fields_s), ("palimpsa_layer_prologue", fields_lp),
                   ("palimpsa_layer_epilogue", fields_le)):
        lines.append(f'printf("%zu\\n", sizeof({st}));')
        for f in fl:
            lines.append(f'printf("%zu\\n", offsetof({st}, {f}));')
    lines.append("return 0;}")
    prog.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.check_call(["gcc", "-std=c99", "-Wall", "-Werror", str(prog), "-o", str(exe)])
    nums = [int(x) for x in subprocess.check_output([str(exe)]).split()]
    it = iter(nums)
    for cls in (L.Problem, L.FwdParams, L.BwdParams, L.Segments, L.LayerPrologue, L.LayerEpilogue):
        assert next(it) == C.sizeof(cls)
        for f in cls._fields_:
            assert next(it) == getattr(cls, f[0]).offset, (cls.__name__, f[0])


def test_version_and_helpers(L):
    lib = L.lib()
    assert lib.palimpsa_abi_version() == L.ABI_VERSION
    assert [lib.palimpsa_padded_k(k) for k in (1, 16, 17, 31, 48, 65, 128, 129, 256, 257)] == \
        [16, 16, 32, 32, 48, 96, 128, 192, 256, 0]
    assert b"workspace" in lib.palimpsa_last_error_string(-5)
    p = L.Problem(num_seqs=3, total_tokens=100)
    assert lib.palimpsa_ckpt_slots(C.byref(p)) == 7 + 3


def test_validation_codes(L):
    lib = L.lib()
    prm = L.FwdParams()
    assert lib.palimpsa_chunk_fwd(C.byref(prm), None) == -8          # struct_size not set
    prm.struct_size = C.sizeof(L.FwdParams)
    assert lib.palimpsa_chunk_fwd(C.byref(prm), None) == -2          # empty shapes
    prm.p.num_seqs, prm.p.seq_len, prm.p.total_tokens = 1, 4, 4
    prm.p.H, prm.p.K, prm.p.V = 1, 512, 8
    assert lib.palimpsa_chunk_fwd(C.byref(prm), None) == -3          # K too large
    prm.p.K = 8
    prm.p.io_dtype = 7
    assert lib.palimpsa_chunk_fwd(C.byref(prm), None) == -4
    prm.p.io_dtype = 0
    assert lib.palimpsa_chunk_fwd(C.byref(prm), None) == -1          # NULL tensors
    b = L.BwdParams()
    b.struct_size = C.sizeof(L.BwdParams)
    assert lib.palimpsa_chunk_bwd(C.byref(b), None) == -2


def test_peer_and_relay_entry_points_validate_before_any_launch(L):
    """Argument checks of the multi-GPU hand-over entry points return their codes without touching a device."""
    lib = L.lib()
    assert lib.palimpsa_peer_wait(None, 1, 1, None, None) == L.E_NULL
    assert lib.palimpsa_peer_signal(None, 1, None) == L.E_NULL
    assert lib.palimpsa_peer_wait(0x1004, 1, 1, None, None) == L.E_ALIGN      # flags are 8-byte aligned
    assert lib.palimpsa_peer_signal(0x1004, 1, None) == L.E_ALIGN
    p, sg = L.Problem(), L.Segments()
    assert lib.palimpsa_cp_relay_prepare(C.byref(p), C.byref(sg), 0, None, None, None) == L.E_NULL
    assert lib.palimpsa_cp_relay(C.byref(p), C.byref(sg), None, None, None, None, None, None, None) == L.E_NULL
    assert lib.palimpsa_cp_relay_prepare(C.byref(p), C.byref(sg), 0, 0x1000, 0x2000, None) == -2   # empty shapes
    assert lib.palimpsa_bwd_tile_rows(128, 128, L.BF16, 0) == 22 and lib.palimpsa_bwd_tile_rows(0, 8, L.BF16, 0) == 0


def test_python_wrappers_reject_cpu_tensors_and_bad_shapes():
    import torch
    from palimpsa_b200.ops import chunk_palimpsa, fused_recurrent_palimpsa
    q = torch.randn(2, 8, 2, 4)
    v = torch.randn(2, 8, 2, 4)
    gt = torch.rand(2, 8, 2)
    g = torch.ones(2)
    with pytest.raises(RuntimeError, match="no CPU path"):
        chunk_palimpsa(q, q, v, v, gt, g, g)
    cu = torch.tensor([0, 8, 16], dtype=torch.int32)
    with pytest.raises(ValueError, match="Batch size must be 1"):
        chunk_palimpsa(q, q, v, v, gt, g, g, cu_seqlens=cu)
    with pytest.raises(ValueError, match="expected to be 1"):
        fused_recurrent_palimpsa(q, q, v, v, gt, g, g, cu_seqlens=cu)
    q1 = q.reshape(1, 16, 2, 4)
    with pytest.raises(ValueError, match="Initial states mismatch"):
        fused_recurrent_palimpsa(q1, q1, v.reshape(1, 16, 2, 4), v.reshape(1, 16, 2, 4), gt.reshape(1, 16, 2), g, g,
                                 cu_seqlens=cu, initial_mu_state=torch.zeros(3, 2, 4, 4),
                                 initial_I_state=torch.ones(3, 2, 4, 4))


def test_naive_ref_matches_fixture():
    import torch
    from oracle import palimpsa_oracle as orc
    from palimpsa_b200.ops import palimpsa_ref
    from tests.helpers import load_golden
    inp, out, meta = load_golden("check_style_unc")
    (o, ov), mu, I = palimpsa_ref(inp["q"], inp["k"], inp["v"], inp["b"], inp["gt"], inp["g"], inp["Ip"], scale=1.0,
                                  output_final_state=True, output_uncertainty=True)
    for x, n in ((o, "o"), (ov, "o_var"), (mu, "final_mu"), (I, "final_I")):
        assert orc.rel_err(x, out[n]) < 1e-5


def test_install_as_palimpsa_ops():
    import sys
    import palimpsa_b200
    saved = {k: sys.modules.get(k) for k in ("palimpsa.ops", "palimpsa.ops.palimpsa")}
    try:
        palimpsa_b200.install_as_palimpsa_ops()
        from palimpsa.ops.palimpsa import chunk_palimpsa as a  # noqa
        from palimpsa.ops import fused_recurrent_palimpsa as b2, palimpsa_ref as c  # noqa
        assert a is palimpsa_b200.chunk_palimpsa
    finally:
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v
