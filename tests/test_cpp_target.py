"""The C++ side of the boundary (include/pyre_b200_target.hpp, the reference's spec::Target over the C ABI): it compiles with a plain
C++17 compiler against the public header alone, every library symbol it needs is exported, and on a GPU it gives what the ctypes mirror
gives on the same handles."""
import ctypes as C
import shutil
import subprocess
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
SHIM = ROOT / "tests" / "cpp" / "target_shim.cpp"


def _compile(tmp_path, shared):
    gxx = shutil.which("g++")
    if not gxx:
        pytest.skip("no g++")
    out = tmp_path / ("libtarget_shim.so" if shared else "target_shim.o")
    cmd = [gxx, "-std=c++17", "-Wall", "-Wextra", "-Werror", "-O1", "-fPIC", "-I", str(ROOT / "include")]
    cmd += ["-shared", str(SHIM), "-o", str(out)] if shared else ["-c", str(SHIM), "-o", str(out)]
    subprocess.run(cmd, check=True)
    return out


def test_adapter_compiles_and_its_symbols_are_exported(tmp_path):
    import pyre_b200 as pb
    obj = _compile(tmp_path, False)
    und = subprocess.run(["nm", "-u", str(obj)], check=True, capture_output=True, text=True).stdout.split()
    need = sorted({s for s in und if s.startswith("pb_")})
    assert {"pb_forward", "pb_verify", "pb_keep", "pb_caps_get", "pb_draft_sampled", "pb_model_cfg"} <= set(need)
    lib = C.CDLL(str(pb.LIB_PATH))
    for s in need:
        assert hasattr(lib, s), s


@pytest.mark.gpu
def test_adapter_matches_the_ctypes_mirror(ctx, tmp_path):
    import pyre_b200 as pb
    from pyre_b200 import synth
    from helpers import small_cfg
    from test_mtp_gpu import _build, WINDOW

    C.CDLL(str(pb.LIB_PATH), mode=C.RTLD_GLOBAL)          # the shim leaves the library's symbols undefined
    shim = C.CDLL(str(_compile(tmp_path, True)))
    shim.shim_make.restype = C.c_void_p
    shim.shim_make.argtypes = [C.c_void_p] * 3
    for f in (shim.shim_free, shim.shim_caps, shim.shim_step, shim.shim_verify, shim.shim_keep, shim.shim_draft):
        f.argtypes = None
    cfg, m, om, mats, cfg_d, dm, odm, dmats, ids = _build(ctx)
    a, b = m.new_state(1), m.new_state(1)
    a.attach_drafter(dm, ids); b.attach_drafter(dm, ids)
    t = shim.shim_make(ctx.h, m.h, a.h)
    assert t
    cv, mw = C.c_int(), C.c_longlong()
    shim.shim_caps(C.c_void_p(t), C.byref(cv), C.byref(mw))
    assert cv.value == 1 and mw.value == m.caps().max_window
    V = cfg.vocab
    prompt = [700, 701, 702, 703, 704]
    lg = np.zeros(V, np.float32)
    for tok in prompt:                                    # step = Model::forward of one token
        assert shim.shim_step(C.c_void_p(t), C.c_uint(tok), lg.ctypes.data_as(C.c_void_p), V) == 0
        ref = b.forward(np.array([tok], np.uint32))[0]
        assert np.array_equal(lg, ref)
    pending = int(lg.argmax())
    hist = (C.c_uint * (len(prompt) + 1))(*prompt, pending)
    out_ids = (C.c_uint * 4)(); qn = (C.c_int * 4)()
    n = shim.shim_draft(C.c_void_p(t), hist, len(prompt) + 1, 3, C.c_float(0.0), 0, out_ids, qn)
    g_ids, _ = b.draft(pending, 3, 0.0)
    assert n == len(g_ids) == 3 and list(out_ids)[:n] == g_ids.tolist() and list(qn)[:n] == [0, 0, 0]
    n2 = shim.shim_draft(C.c_void_p(t), hist, len(prompt) + 1, 3, C.c_float(0.0), 1, out_ids, qn)
    assert n2 == 3 and list(qn)[:3] == [2, 2, 2] and list(out_ids)[:3] != g_ids.tolist()       # drawn by the sampler, distributions attached
    win = np.array([pending] + g_ids.tolist(), np.uint32)
    lw = np.zeros((len(win), V), np.float32)
    assert shim.shim_verify(C.c_void_p(t), win.ctypes.data_as(C.c_void_p), len(win), lw.ctypes.data_as(C.c_void_p), V) == 0
    assert np.array_equal(lw, b.forward_multi(win))
    assert shim.shim_keep(C.c_void_p(t), len(win), 2) == 0
    b.spec_keep(len(win), 2)
    assert a.pos() == b.pos() == len(prompt) + 2
    assert shim.shim_keep(C.c_void_p(t), len(win), 1) == pb.PB_ERR_STATE                      # no window pending: the library's status comes through
    plain = m.new_state(1)                                                                     # no drafter: the n-gram drafter's turn
    t2 = shim.shim_make(ctx.h, m.h, plain.h)
    plain.forward(np.array(prompt, np.uint32))
    assert shim.shim_draft(C.c_void_p(t2), hist, len(prompt) + 1, 3, C.c_float(0.0), 0, out_ids, qn) == -1
    shim.shim_free(C.c_void_p(t)); shim.shim_free(C.c_void_p(t2))
    for s in (a, b, plain):
        s.destroy()
