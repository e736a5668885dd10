#!/usr/bin/env python3
"""Golden vectors for the gated attention of the token loop from Hugging Face transformers' Qwen3-Next code.

    python tests/golden/make_hf_attention_golden.py       # needs torch and transformers >= 4.57 (CPU is enough)

writes tests/golden/hf_gated_attention.npz.  What is taken from transformers: the zero-centred RMS norm of q and k
(Qwen3NextRMSNorm: x * rsqrt(mean x^2 + eps) * (1 + w)), the partial rotary embedding (apply_rotary_pos_emb /
rotate_half on the first n_rot dims), grouped-query causal attention (eager_attention_forward: softmax in f32 of
q.k / sqrt(hd)) and the sigmoid output gate that rides in the query projection (Qwen3NextAttention.forward).  The
reference computes the same (attn_core, src/model/qwen4exp_gguf.rs:1558-1615; its GGUF stores the norm weights already
as 1 + w, which is what the vectors hold).  Stored: per token the projected rows qf [n_head][q(hd) | gate(hd)], kf, vf,
the folded norm weights, rope base / n_rot, and the attention output rows [t][n_head * hd] (after the gate, before o_proj).
"""
from pathlib import Path

import numpy as np
import torch
from transformers.models.qwen3_next import modeling_qwen3_next as mq

NH, NKV, HD, NROT, T, BASE, EPS = 4, 2, 256, 64, 10, 1e7, 1e-6


def main():
    g = torch.Generator().manual_seed(777)
    qf = torch.randn(1, T, NH, 2 * HD, generator=g)                 # per head: query | gate
    kf = torch.randn(1, T, NKV, HD, generator=g)
    vf = torch.randn(1, T, NKV, HD, generator=g)
    qn, kn = mq.Qwen3NextRMSNorm(HD, eps=EPS), mq.Qwen3NextRMSNorm(HD, eps=EPS)
    with torch.no_grad():
        qn.weight.copy_(0.1 * torch.randn(HD, generator=g)); kn.weight.copy_(0.1 * torch.randn(HD, generator=g))
    query, gate = torch.chunk(qf, 2, dim=-1)
    gate = gate.reshape(1, T, NH * HD)
    with torch.no_grad():
        q = qn(query).transpose(1, 2)                               # [1][NH][T][HD]
        k = kn(kf).transpose(1, 2)
    v = vf.transpose(1, 2)
    inv_freq = 1.0 / (BASE ** (torch.arange(0, NROT, 2, dtype=torch.float32) / NROT))
    freqs = torch.arange(T, dtype=torch.float32)[:, None] * inv_freq[None, :]
    emb = torch.cat((freqs, freqs), dim=-1)[None]                   # [1][T][NROT]
    q, k = mq.apply_rotary_pos_emb(q, k, emb.cos(), emb.sin())

    class Shim(torch.nn.Module):
        num_key_value_groups = NH // NKV
        training = False
    mask = torch.full((T, T), float("-inf")).triu(1)[None, None]
    out, _ = mq.eager_attention_forward(Shim(), q, k, v, mask, scaling=HD ** -0.5)
    out = out.reshape(1, T, NH * HD) * torch.sigmoid(gate)
    dst = Path(__file__).resolve().parent / "hf_gated_attention.npz"
    np.savez_compressed(dst, n_head=NH, n_kv=NKV, hd=HD, n_rot=NROT, t=T, rope_base=BASE, eps=EPS,
                        qf=qf[0].reshape(T, NH * 2 * HD).numpy(), kf=kf[0].reshape(T, NKV * HD).numpy(), vf=vf[0].reshape(T, NKV * HD).numpy(),
                        q_norm=(1.0 + qn.weight.detach()).numpy(), k_norm=(1.0 + kn.weight.detach()).numpy(), att=out[0].detach().numpy().astype(np.float32))
    print("wrote", dst, tuple(out.shape))


if __name__ == "__main__":
    main()
