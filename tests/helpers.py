"""Shared test helpers: realise a synthetic model description in the CPU oracle."""
import numpy as np

import oracle


def oracle_cfg(cfg):
    """Copy a pyre_b200.Cfg (same field layout) into the oracle's config struct."""
    oc = oracle.Cfg()
    for name, _ in oracle.Cfg._fields_:
        setattr(oc, name, getattr(cfg, name))
    return oc


def oracle_model(cfg, spec, seed=0):
    om = oracle.Model(oracle_cfg(cfg))
    mats = {}
    for item in spec:
        if item[0] == "mat":
            _, layer, role, t, rows, cols, tid = item
            q = oracle.QMat.synth(t, rows, cols, seed, tid)
            om.set_mat(layer, role, q)
            mats[(layer, role)] = q
        else:
            _, layer, role, arr = item
            om.set_vec(layer, role, arr)
            mats[(layer, role)] = np.asarray(arr, dtype=np.float32)
    return om, mats


def small_cfg(pb, **kw):
    """A scaled-down hybrid config that keeps every structural feature of the full model."""
    base = dict(n_layers=4, d=512, n_head=4, n_kv=2, hd=256, n_rot=64, n_exp=16, top_k=4, ff_exp=256, ff_sh=256,
                lin_nk=2, lin_nv=4, lin_dk=128, lin_dv=128, conv_k=4, full_every=4, vocab=1024, max_ctx=512,
                kv_bits=0, kv_recent=64)
    base.update(kw)
    return pb.make_cfg(**base)
