"""Writes tests/golden/hf_yarn.npz: YaRN inverse rope frequencies and the attention factor (mscale) computed with
Hugging Face transformers' `_compute_yarn_parameters` for a few (n_rot, base, trained context, context) cases.

    python tests/golden/make_hf_yarn_golden.py

The reference builds its scaled table in src/qn_ctx.rs:160-186 with the same defaults (beta_fast 32, beta_slow 1,
correction range floored / ceiled, mscale = 1 + 0.1 ln(scale)) but blends the two regimes the other way round:
index i gets  interp * (1 - ramp) + extrap * ramp  where transformers (and llama.cpp) compute
interp * ramp + extrap * (1 - ramp).  The oracle follows the reference; the test holds it to these vectors through
    oracle_inv[i] + hf_inv[i] == extrap[i] * (1 + 1 / scale),
which pins the correction range, the ramp and mscale, and records the difference.
"""
from pathlib import Path

import numpy as np
from transformers import PretrainedConfig
from transformers import modeling_rope_utils as R

CASES = [(64, 1e7, 4096, 16384), (64, 1e7, 262144, 1048576), (128, 1e6, 32768, 131072), (64, 1e4, 2048, 3000), (64, 1e7, 1024, 4096)]


def hf(n_rot, base, ctx_train, ctx):
    cfg = PretrainedConfig()
    cfg.rope_theta = base
    cfg.head_dim = n_rot
    cfg.hidden_size = n_rot
    cfg.num_attention_heads = 1
    cfg.max_position_embeddings = ctx
    cfg.partial_rotary_factor = 1.0
    cfg.rope_parameters = {"rope_type": "yarn", "factor": ctx / ctx_train, "original_max_position_embeddings": ctx_train, "rope_theta": base}
    inv, att = R._compute_yarn_parameters(cfg, device="cpu")
    return inv.numpy().astype(np.float32), float(att)


def main():
    out = {"cases": np.array(CASES, dtype=np.float64)}
    for i, (n_rot, base, tr, ctx) in enumerate(CASES):
        inv, att = hf(n_rot, base, tr, ctx)
        out[f"inv{i}"] = inv
        out[f"att{i}"] = np.float32(att)
    np.savez(Path(__file__).parent / "hf_yarn.npz", **out)


if __name__ == "__main__":
    main()
