#!/usr/bin/env python3
"""Golden vectors for the Gated DeltaNet recurrence from an independent implementation: Hugging Face transformers'
Qwen3-Next (`torch_recurrent_gated_delta_rule`, `l2norm`, the causal depthwise conv + SiLU of Qwen3NextGatedDeltaNet).

    python tests/golden/make_hf_deltanet_golden.py        # needs torch and transformers >= 4.57 (CPU is enough)

writes tests/golden/hf_gated_deltanet.npz.  The model family of the reference (qwen4exp) shares with Qwen3-Next the conv,
the L2 norms with q scaled by 1/sqrt(dk), the gates g = exp(-exp(A_log) * softplus(a + dt_bias)) and beta = sigmoid(b),
and the delta rule itself; it differs in two places that this script lines up by hand:
  * V head h reads K head h % nk (src/model/qwen4exp_gguf.rs:1655), where Qwen3-Next repeats K heads in blocks
    (h // (nv / nk)) -- the q and k handed to the transformers function are gathered with the reference's rule;
  * the output gate is sigmoid(z) (:1667), not SiLU(z) -- so the vectors stop at the readout before the gated norm
    (the test applies a weight-1 RMS norm with z = +30, i.e. gate 1, on both sides).
Stored: the inputs (projections qkv [t][ch], beta and alpha pre-activations, ssm_a = -exp(A_log), dt_bias, conv weights)
and, from transformers, the readout [t][nv][dv] and the final recurrent state [nv][dk][dv].
"""
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F
from transformers.models.qwen3_next import modeling_qwen3_next as mq

NK, NV, DK, DV, K, T = 2, 4, 128, 128, 4, 12


def main():
    g = torch.Generator().manual_seed(20240607)
    ch = 2 * NK * DK + NV * DV
    qkv = torch.randn(T, ch, generator=g)
    b_raw = torch.randn(T, NV, generator=g)
    a_raw = torch.randn(T, NV, generator=g)
    A_log = 0.5 * torch.randn(NV, generator=g)
    dt_bias = torch.randn(NV, generator=g)
    conv_w = 0.5 * torch.randn(ch, K, generator=g)
    # causal depthwise conv + SiLU as Qwen3NextGatedDeltaNet.forward does it without a cache: conv1d with padding K-1, cut to T
    x = qkv.t().unsqueeze(0)                                        # [1][ch][T]
    mixed = F.silu(F.conv1d(x, conv_w.unsqueeze(1), bias=None, padding=K - 1, groups=ch)[:, :, :T]).transpose(1, 2)   # [1][T][ch]
    q, k, v = torch.split(mixed, [NK * DK, NK * DK, NV * DV], dim=-1)
    q = q.reshape(1, T, NK, DK); k = k.reshape(1, T, NK, DK); v = v.reshape(1, T, NV, DV)
    kh = torch.arange(NV) % NK                                      # the reference's head map
    q, k = q[:, :, kh], k[:, :, kh]                                 # [1][T][NV][DK]
    beta = b_raw.sigmoid().unsqueeze(0)
    gdec = (-A_log.float().exp() * F.softplus(a_raw.float() + dt_bias)).unsqueeze(0)
    out, state = mq.torch_recurrent_gated_delta_rule(q, k, v, g=gdec, beta=beta, initial_state=None, output_final_state=True,
                                                     use_qk_l2norm_in_kernel=True)
    dst = Path(__file__).resolve().parent / "hf_gated_deltanet.npz"
    np.savez_compressed(dst, nk=NK, nv=NV, dk=DK, dv=DV, conv_k=K, t=T,
                        qkv=qkv.numpy(), beta_raw=b_raw.numpy(), alpha_raw=a_raw.numpy(), ssm_a=(-A_log.exp()).numpy(), dt_bias=dt_bias.numpy(),
                        conv_w=conv_w.numpy(), readout=out[0].numpy().astype(np.float32), state=state[0].numpy().astype(np.float32))
    print("wrote", dst, "readout", tuple(out.shape), "state", tuple(state.shape))


if __name__ == "__main__":
    main()
