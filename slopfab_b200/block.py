"""One DiT block on top of the quantized-Linear path (the caller side of the path).

Order of operations of the reference's ``run_block`` (src/dit/transformer_execution.cpp:247-455):

    n1 = modulate(rmsnorm(x, norm1), scale_msa, shift_msa)      fused with the fp4 quantizer, ONE pass
    q, k, v = n1 Wq^T, n1 Wk^T, n1 Wv^T                         three NVFP4 GEMMs on one quantized n1
    attention(q, k, v)                                          bf16 tcgen05 kernel of this library on the thirds of the
                                                                fused projection as they lie (or a callable you pass)
    x += gate_msa * (attn Wo^T)                                 NVFP4 Linear, gated residual in its epilogue
    n2 = modulate(rmsnorm(x, norm2), scale_mlp, shift_mlp)      fused with the fp4 quantizer
    x += gate_mlp * (act(n2 W1^T) W2^T)                         GELU-tanh fused in the first GEMM's epilogue

Head-wise q/k RMSNorm and MM-RoPE sit between the projections and attention (QK-norm first, then RoPE; v untouched):
one in-place pass per third of the fused projection, run when the weights carry q_norm / k_norm or `rope` is given.
The FFN is the plain GELU form of the benchmark configuration by default; `ffn_form="swiglu"` runs the reference's H3
form instead (src/dit/transformer_execution.cpp:433-441): fc1 is the fused [gate | up] weight with 2 * ffn rows and the
SwiGLU epilogue writes silu(gate) * up, ffn columns wide, so the [rows, 2 * ffn] intermediate never exists.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from . import (ACT_GELU_TANH, ACT_NONE, ACT_SWIGLU, F32, NVFP4_ACT_GEMM_FEED, Epilogue, Norm, check, lib, ptr, stream_ptr)


@dataclass
class Nvfp4Linear:
    data: torch.Tensor    # u8 [N, K/2]
    scale: torch.Tensor   # u8 [N*K/16], 128x4-tiled
    global_scale: float
    out_features: int
    in_features: int

    @staticmethod
    def random(out_features: int, in_features: int, device="cuda", seed: int = 0) -> "Nvfp4Linear":
        """Random nibbles with block scales around 2^-1..2^1 and a global scale that gives N(0, 0.02)-like weights."""
        g = torch.Generator(device=device).manual_seed(seed)
        data = torch.randint(0, 256, (out_features, in_features // 2), dtype=torch.uint8, device=device, generator=g)
        scale = torch.randint(0x30, 0x40, (out_features * in_features // 16,), dtype=torch.uint8, device=device, generator=g)
        return Nvfp4Linear(data, scale, 0.02 / 2.5, out_features, in_features)


@dataclass
class BlockWeights:
    qkv: Nvfp4Linear      # [3*hidden, hidden]
    out: Nvfp4Linear
    fc1: Nvfp4Linear
    fc2: Nvfp4Linear
    norm1: torch.Tensor   # bf16 [hidden]
    norm2: torch.Tensor
    q_norm: torch.Tensor | None = None   # bf16 [128]: RMSNorm over the head dimension of q (and k_norm of k)
    k_norm: torch.Tensor | None = None


class Nvfp4Block:
    """Scratch and launch plumbing for blocks of one geometry."""

    def __init__(self, rows: int, hidden: int, heads: int, ffn: int, device="cuda", ffn_form: str = "gelu"):
        if ffn_form not in ("gelu", "swiglu"):
            raise ValueError("ffn_form must be 'gelu' or 'swiglu'")
        self.rows, self.hidden, self.heads, self.ffn, self.ffn_form = rows, hidden, heads, ffn, ffn_form
        kmax = max(hidden, ffn)
        self.xq = torch.empty((rows, kmax // 2), dtype=torch.uint8, device=device)
        self.xs = torch.empty(lib.sfq_nvfp4_act_scale_bytes(rows, kmax), dtype=torch.uint8, device=device)
        self.qkv = torch.empty((rows, 3 * hidden), dtype=torch.bfloat16, device=device)
        self.branch = torch.empty((rows, hidden), dtype=torch.bfloat16, device=device)
        self.h = torch.empty((rows, ffn), dtype=torch.bfloat16, device=device)
        self.linear_ms = 0.0
        self.attn = torch.empty((rows, hidden), dtype=torch.bfloat16, device=device)
        self.attn_ws = None  # V transposed, allocated on first use of the library's own attention
        # True: x += gate * branch inside the out / fc2 GEMM epilogues (same bits; measured 3 % slower per block than the
        # separate add_gated kernel at 75600 tokens, because the single-accumulator nvfp4 epilogue then waits on x)
        self.fuse_residual = False

    def _quantize(self, x, dim, norm: Norm | None):
        check(lib.sfq_quantize_nvfp4_block(ptr(x), C.byref(norm) if norm is not None else None, ptr(self.xq), ptr(self.xs),
                                           None, self.rows, dim, NVFP4_ACT_GEMM_FEED, stream_ptr()))

    def _gemm(self, w: Nvfp4Linear, y, act=ACT_NONE, gate=None, gate_index=None):
        """y = act(x W^T), or with `gate`: y += gate[gate_index] * (x W^T) fused in the epilogue."""
        ep = Epilogue(None, None, w.global_scale, None, F32, act, ptr(gate) if gate is not None else None,
                      ptr(gate_index) if gate is not None else None)
        check(lib.sfq_gemm_nvfp4(ptr(self.xq), ptr(self.xs), ptr(w.data), ptr(w.scale), C.byref(ep), ptr(y), self.rows,
                                 w.out_features, w.in_features, stream_ptr()))

    def forward(self, x: torch.Tensor, w: BlockWeights, mod: dict, adaln_index: torch.Tensor, eps: float = 1e-5,
                attention=None, time_linears: bool = False, rope=None) -> torch.Tensor:
        """x bf16 [rows, hidden] is updated in place and returned. `mod` holds fp32 [T*3, hidden] tables
        scale_msa, shift_msa, gate_msa, scale_mlp, shift_mlp, gate_mlp; adaln_index int32 [rows]."""
        rows, hidden, heads = self.rows, self.hidden, self.heads
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)] if time_linears else None
        if ev:
            ev[0].record()
        n1 = Norm(ptr(w.norm1), ptr(mod["scale_msa"]), ptr(mod["shift_msa"]), ptr(adaln_index), eps)
        self._quantize(x, hidden, n1)
        self._gemm(w.qkv, self.qkv)
        if ev:
            ev[1].record()
        if w.q_norm is not None or w.k_norm is not None or rope is not None:
            cos, sin = (ptr(rope[0]), ptr(rope[1])) if rope is not None else (None, None)  # fp32 [rows, 96] each
            for third, nw in ((0, w.q_norm), (1, w.k_norm)):
                if nw is not None or rope is not None:
                    check(lib.sfq_head_norm_rope(self.qkv.data_ptr() + third * hidden * 2, 3 * hidden, ptr(nw) if nw is not None else None,
                                                 cos, sin, rows, heads, hidden // heads, eps, stream_ptr()))
        if attention is None:
            # q, k, v are the column thirds of self.qkv (row pitch 3 * hidden): no split, no transpose
            if hidden != heads * 128:
                raise ValueError("the attention kernel is built for head_dim 128")
            if self.attn_ws is None:
                n = C.c_size_t()
                check(lib.sfq_attention_workspace_bytes(rows, heads, 128, C.byref(n)))
                self.attn_ws = torch.empty(n.value, dtype=torch.uint8, device=x.device)
            base = self.qkv.data_ptr()
            check(lib.sfq_attention_forward(base, 3 * hidden, base + 2 * hidden, base + 4 * hidden, 3 * hidden, ptr(self.attn), hidden,
                                            rows, rows, heads, heads, 128, 0.0, ptr(self.attn_ws), self.attn_ws.numel(), stream_ptr()))
            attn = self.attn
        else:
            q, k, v = (t.view(1, rows, heads, hidden // heads).transpose(1, 2) for t in self.qkv.split(hidden, dim=1))
            attn = attention(q, k, v).transpose(1, 2).reshape(rows, hidden).contiguous()
        if ev:
            ev[2].record()
        self._quantize(attn, hidden, None)
        if self.fuse_residual:
            self._gemm(w.out, x, gate=mod["gate_msa"], gate_index=adaln_index)
        else:
            self._gemm(w.out, self.branch)
            check(lib.sfq_add_gated(ptr(x), ptr(self.branch), ptr(mod["gate_msa"]), ptr(adaln_index), rows, hidden, stream_ptr()))
        n2 = Norm(ptr(w.norm2), ptr(mod["scale_mlp"]), ptr(mod["shift_mlp"]), ptr(adaln_index), eps)
        self._quantize(x, hidden, n2)
        if self.ffn_form == "swiglu":
            if w.fc1.out_features != 2 * self.ffn:
                raise ValueError("the SwiGLU form needs fc1 = [gate | up] with 2 * ffn rows")
            self._gemm(w.fc1, self.h, ACT_SWIGLU)
        else:
            self._gemm(w.fc1, self.h, ACT_GELU_TANH)
        self._quantize(self.h, self.ffn, None)
        if self.fuse_residual:
            self._gemm(w.fc2, x, gate=mod["gate_mlp"], gate_index=adaln_index)
        else:
            self._gemm(w.fc2, self.branch)
            check(lib.sfq_add_gated(ptr(x), ptr(self.branch), ptr(mod["gate_mlp"]), ptr(adaln_index), rows, hidden, stream_ptr()))
        if ev:
            ev[3].record()
            ev[3].synchronize()
            self.linear_ms += ev[0].elapsed_time(ev[1]) + ev[2].elapsed_time(ev[3])
        return x
