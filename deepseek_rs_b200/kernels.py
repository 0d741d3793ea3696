"""Host-side mirror of the reference's kernel call surface for the routed-expert path, over torch CUDA tensors.

Method names and operand order follow the reference's generated launch methods (``engine.kernels.moe.<kernel>`` and
``engine.kernels.quantize.q8k_quantize``; engine/src/session.rs:2038-2153) minus the LaunchConfig, which the library
chooses itself, and minus the lookup tables, which live inside the library. Every call goes through the C ABI of
libdsmoe.so on the current torch stream and raises ``DsmoeError`` on a non-zero status. torch is only the owner of
device memory and streams here.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from .formats import IQ2XXS_BYTES, Q2K_BYTES, Q8K_BYTES, QK_K

LAYOUT_NATIVE, LAYOUT_ROWSOA = _lib.LAYOUT_NATIVE, _lib.LAYOUT_ROWSOA


class DsmoeError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"dsmoe status {code}: {msg}")
        self.code = code


def _ptr(t):
    if t is None:
        return None
    assert t.is_cuda and t.is_contiguous(), "dsmoe operands must be contiguous CUDA tensors"
    return C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


class MoeKernels:
    """One library handle on one device: the counterpart of ``Kernels::load`` (engine/src/engine.rs:31-54)."""

    def __init__(self, device: int = 0, n_embd: int = 4096, n_ff: int = 2048, n_expert: int = 256,
                 n_expert_used: int = 6, swiglu_clamp: float = 10.0, route_scale: float = 1.5, f16_ieee: bool = False,
                 max_tokens: int = 64, max_layers: int = 1):
        self.lib = _lib.load()
        if not torch.cuda.is_available():
            raise RuntimeError("dsmoe needs a CUDA device; there is no CPU path")
        self.cfg = _lib.Config(n_embd, n_ff, n_expert, n_expert_used, swiglu_clamp, route_scale, int(f16_ieee),
                               max_tokens, max_layers)
        self.device = device
        torch.cuda.set_device(device)
        h = C.c_void_p()
        rc = self.lib.dsmoe_create(C.byref(self.cfg), device, C.byref(h))
        if rc != 0:
            raise DsmoeError(rc, "dsmoe_create failed (needs a compute-capability 10.x device)")
        self.h = h

    def close(self):
        if getattr(self, "h", None):
            self.lib.dsmoe_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc: int):
        if rc != 0:
            raise DsmoeError(rc, self.lib.dsmoe_last_error(self.h).decode())

    def device_status(self) -> int:
        """Synchronises the current stream and returns the device status word (0 = no bounded wait ever expired);
        raises DsmoeError otherwise."""
        code = C.c_int(0)
        self._check(self.lib.dsmoe_device_status(self.h, _stream(), C.byref(code)))
        return code.value

    def set_phase_events(self, events):
        """Six torch.cuda.Event(enable_timing=True), already recorded once, or None to clear: the batched path records
        them between its phases."""
        if not events:
            self._check(self.lib.dsmoe_set_phase_events(self.h, None, 0))
            return
        arr = (C.c_void_p * 6)(*[C.c_void_p(e.cuda_event) for e in events])
        self._check(self.lib.dsmoe_set_phase_events(self.h, arr, 6))

    def debug_set(self, what: int, value: int):
        """Test hook for the bounded-wait error path (see dsmoe_debug_set in include/dsmoe.h)."""
        self._check(self.lib.dsmoe_debug_set(self.h, what, value))

    @property
    def launch_count(self) -> int:
        return int(self.lib.dsmoe_launch_count(self.h))

    # ---- tier 1: one method per reference kernel ---------------------------------------------------------------

    def q8k_quantize(self, x, out, in_dim: int, n_rows: int):
        """engine/src/kernels/quantize.rs:309 — x f32 [n_rows, in_dim] -> out uint8 Q8_K blocks."""
        self._check(self.lib.dsmoe_q8k_quantize(self.h, _stream(), _ptr(x), _ptr(out), in_dim, n_rows))

    def router_select_parallel(self, logits, bias, hash, tokens, probs, selected, weights, token_scalar: int,
                               hash_rows: int, n_tokens: int, has_bias: int, hash_mode: int):
        """engine/src/kernels/moe.rs:177"""
        self._check(self.lib.dsmoe_router_select(self.h, _stream(), _ptr(logits), _ptr(bias), _ptr(hash), _ptr(tokens),
                                                 _ptr(probs), _ptr(selected), _ptr(weights), token_scalar, hash_rows,
                                                 n_tokens, has_bias, hash_mode))

    def moe_gate_up_mid_qwarp32(self, gate_base, up_base, xq, selected, weights, gate_out, up_out, mid_out,
                                gate_expert_bytes: int, gate_row_bytes: int, xq_blocks: int, expert_mid_dim: int,
                                n_expert: int, clamp: float, n_tokens: int | None = None, layout: int = LAYOUT_NATIVE):
        """engine/src/kernels/moe.rs:622 — the pair count comes from the launch grid in the reference; here it is
        n_tokens (default: rows of ``selected``)."""
        if n_tokens is None:
            n_tokens = selected.numel() // n_expert
        self._check(self.lib.dsmoe_gate_up_mid(self.h, _stream(), _ptr(gate_base), _ptr(up_base), _ptr(xq),
                                               _ptr(selected), _ptr(weights), _ptr(gate_out), _ptr(up_out),
                                               _ptr(mid_out), gate_expert_bytes, gate_row_bytes, xq_blocks,
                                               expert_mid_dim, n_expert, n_tokens, clamp, layout))

    def moe_down_qwarp32(self, down_base, midq, selected, down_out, down_expert_bytes: int, down_row_bytes: int,
                         midq_blocks: int, out_dim: int, n_expert: int, n_tokens: int | None = None,
                         layout: int = LAYOUT_NATIVE):
        """engine/src/kernels/moe.rs:821"""
        if n_tokens is None:
            n_tokens = selected.numel() // n_expert
        self._check(self.lib.dsmoe_down(self.h, _stream(), _ptr(down_base), _ptr(midq), _ptr(selected), _ptr(down_out),
                                        down_expert_bytes, down_row_bytes, midq_blocks, out_dim, n_expert, n_tokens,
                                        layout))

    def moe_down_sum6_qwarp32(self, down_base, midq, selected, out, down_expert_bytes: int, down_row_bytes: int,
                              midq_blocks: int, out_dim: int, n_expert: int | None = None, n_tokens: int = 1,
                              layout: int = LAYOUT_NATIVE):
        """engine/src/kernels/moe.rs:922 — the reference sums six slots of one token; n_expert / n_tokens generalise."""
        if n_expert is None:
            n_expert = self.cfg.n_expert_used
        self._check(self.lib.dsmoe_down_sum(self.h, _stream(), _ptr(down_base), _ptr(midq), _ptr(selected), _ptr(out),
                                            down_expert_bytes, down_row_bytes, midq_blocks, out_dim, n_expert, n_tokens,
                                            layout))

    def moe_sum(self, down, out, out_dim: int, n_expert: int, n_tokens: int):
        """engine/src/kernels/moe.rs:983"""
        self._check(self.lib.dsmoe_moe_sum(self.h, _stream(), _ptr(down), _ptr(out), out_dim, n_expert, n_tokens))

    # ---- router logits and shared expert (engine/src/session.rs:1894-2008) --------------------------------------

    def quantize_q8_0(self, x, xq, xscale, in_dim: int, n_tokens: int):
        """engine/src/kernels/quantize.rs:147 — x f32 [n_tokens, in_dim] -> int8 codes and f32 scales per 32."""
        self._check(self.lib.dsmoe_quantize_q8_0(self.h, _stream(), _ptr(x), _ptr(xq), _ptr(xscale), in_dim, n_tokens))

    def matmul_q8_0_preq_warp8(self, w, xq, xscale, out, in_dim: int, out_dim: int, n_tokens: int = 1):
        """engine/src/kernels/matmul.rs:357 (n_tokens > 1: its batched twin)."""
        self._check(self.lib.dsmoe_matmul_q8_0(self.h, _stream(), _ptr(w), _ptr(xq), _ptr(xscale), _ptr(out), in_dim,
                                               out_dim, n_tokens))

    def swiglu(self, gate, up, out, n: int, clamp: float, weight: float):
        """engine/src/kernels/utils.rs:141"""
        self._check(self.lib.dsmoe_swiglu(self.h, _stream(), _ptr(gate), _ptr(up), _ptr(out), n, clamp, weight))

    def matmul_f16(self, w, x, out, in_dim: int, out_dim: int, n_tokens: int):
        """engine/src/kernels/matmul.rs:57 — w: f16 bit patterns (uint16 / float16 tensor)."""
        self._check(self.lib.dsmoe_matmul_f16(self.h, _stream(), _ptr(w), _ptr(x), _ptr(out), in_dim, out_dim, n_tokens))

    def shared_expert(self, gate_w, up_w, down_w, x, n_tokens: int, out):
        """The shared expert of engine/src/session.rs:1894-1986 in one call."""
        self._check(self.lib.dsmoe_shared_expert(self.h, _stream(), _ptr(gate_w), _ptr(up_w), _ptr(down_w), _ptr(x),
                                                 n_tokens, _ptr(out)))

    # ---- helpers with no reference kernel ------------------------------------------------------------------------

    def moe_sum_indexed(self, rows, pos, out, out_dim: int, n_expert: int, n_tokens: int):
        """The slot-order sum of engine/src/kernels/moe.rs:983 over rows addressed through ``pos`` (int32)."""
        self._check(self.lib.dsmoe_moe_sum_indexed(self.h, _stream(), _ptr(rows), _ptr(pos), _ptr(out), out_dim, n_expert,
                                                   n_tokens))

    def dequant_iq2xxs(self, blocks, n_blocks: int, out):
        self._check(self.lib.dsmoe_dequant_iq2xxs(self.h, _stream(), _ptr(blocks), n_blocks, _ptr(out)))

    def dequant_q2k(self, blocks, n_blocks: int, out):
        self._check(self.lib.dsmoe_dequant_q2k(self.h, _stream(), _ptr(blocks), n_blocks, _ptr(out)))

    def relayout_iq2xxs(self, src, dst, n_rows: int, blocks_per_row: int, inverse: bool = False):
        self._check(self.lib.dsmoe_relayout_iq2xxs(self.h, _stream(), _ptr(src), _ptr(dst), n_rows, blocks_per_row,
                                                   int(inverse)))

    def relayout_q2k(self, src, dst, n_rows: int, blocks_per_row: int, inverse: bool = False):
        self._check(self.lib.dsmoe_relayout_q2k(self.h, _stream(), _ptr(src), _ptr(dst), n_rows, blocks_per_row,
                                                int(inverse)))

    # ---- FP8 block-scaled projection -------------------------------------------------------------------------

    def fp8_quantize(self, x, codes, scales, rows: int, cols: int, rows_per_block: int):
        self._check(self.lib.dsmoe_fp8_quantize(self.h, _stream(), _ptr(x), _ptr(codes), _ptr(scales), rows, cols,
                                                rows_per_block))

    def fp8_linear(self, a_codes, a_scale, w_codes, w_scale, out_bf16, M: int, N: int, K: int):
        self._check(self.lib.dsmoe_fp8_linear(self.h, _stream(), _ptr(a_codes), _ptr(a_scale), _ptr(w_codes),
                                              _ptr(w_scale), _ptr(out_bf16), M, N, K))

    # ---- tier 2 ---------------------------------------------------------------------------------------------------

    def layer_register(self, layer: int, gate, up, down, layout: int):
        self._check(self.lib.dsmoe_layer_register(self.h, layer, _ptr(gate), _ptr(up), _ptr(down), layout))

    def layer_register_extras(self, layer: int, router_f16=None, router_bias=None, hash_table=None, shared_gate=None,
                              shared_up=None, shared_down=None):
        """The tensors beside the routed experts (router matrix, bias, hash table, shared expert); any may be None."""
        hash_rows = 0 if hash_table is None else hash_table.numel() // self.cfg.n_expert_used
        self._check(self.lib.dsmoe_layer_register_extras(self.h, layer, _ptr(router_f16), _ptr(router_bias),
                                                         _ptr(hash_table), hash_rows, _ptr(shared_gate), _ptr(shared_up),
                                                         _ptr(shared_down)))

    def ffn_forward(self, layer: int, x, routed_out, logits=None, tokens=None, token_scalar: int = 0, hash_mode: int = 0,
                    shared_out=None, residual_hc=None, hc_split=None, out_hc=None, selected_out=None, weights_out=None):
        """Steps g, h, i of Session::decode_attn_out_and_ffn (engine/src/session.rs:1894-2180) in one call. x: f32 or
        bfloat16 [T, n_embd]."""
        p = lambda t: None if t is None else t.data_ptr()
        a = _lib.FfnArgs()
        a.x, a.x_dtype, a.n_tokens = p(x), (_lib.DTYPE_BF16 if x.dtype == torch.bfloat16 else _lib.DTYPE_F32), x.shape[0]
        a.logits, a.tokens, a.token_scalar, a.hash_mode = p(logits), p(tokens), token_scalar, hash_mode
        a.routed_out, a.shared_out = p(routed_out), p(shared_out)
        a.residual_hc, a.hc_split, a.out_hc = p(residual_hc), p(hc_split), p(out_hc)
        if out_hc is not None:
            a.n_hc, a.mix_hc = residual_hc.shape[1], hc_split.shape[1]
        a.selected_out, a.weights_out = p(selected_out), p(weights_out)
        for t in (x, logits, tokens, routed_out, shared_out, residual_hc, hc_split, out_hc, selected_out, weights_out):
            assert t is None or (t.is_cuda and t.is_contiguous())
        self._check(self.lib.dsmoe_ffn_forward(self.h, _stream(), layer, C.byref(a)))

    def hc_split_weighted_sum_norm_fused(self, mix, scale, base, residual_hc, norm_w, split, out, norm_out, n_embd: int,
                                         n_hc: int, n_rows: int, sinkhorn_iters: int, epsv: float, norm_eps: float):
        """engine/src/kernels/hc.rs:313 - the producer of ffn_norm"""
        self._check(self.lib.dsmoe_hc_split_weighted_sum_norm(self.h, _stream(), _ptr(mix), _ptr(scale), _ptr(base),
                                                              _ptr(residual_hc), _ptr(norm_w), _ptr(split), _ptr(out),
                                                              _ptr(norm_out), n_embd, n_hc, n_rows, sinkhorn_iters, epsv,
                                                              norm_eps))

    def hc_expand(self, block_out, block_add, residual_hc, split, out_hc, n_embd: int, n_hc: int, n_tokens: int,
                  mix_hc: int, has_add: int):
        """engine/src/kernels/hc.rs:212"""
        self._check(self.lib.dsmoe_hc_expand(self.h, _stream(), _ptr(block_out), _ptr(block_add), _ptr(residual_hc),
                                             _ptr(split), _ptr(out_hc), n_embd, n_hc, n_tokens, mix_hc, has_add))

    def moe_forward(self, layer: int, x, logits, n_tokens: int, out, selected_out=None, weights_out=None):
        self._check(self.lib.dsmoe_moe_forward(self.h, _stream(), layer, _ptr(x), _ptr(logits), n_tokens, _ptr(out),
                                               _ptr(selected_out), _ptr(weights_out)))

    def expert_ffn(self, layer: int, xq, selected, weights, n_tokens: int, out):
        """Rows already routed and Q8_K-quantised -> slot-summed expert output (what an expert-parallel rank runs)."""
        self._check(self.lib.dsmoe_expert_ffn(self.h, _stream(), layer, _ptr(xq), _ptr(selected), _ptr(weights),
                                              n_tokens, _ptr(out)))

    def moe_forward_host(self, layer: int, x_host, logits_host, n_tokens: int, out_host, selected_host=None,
                         weights_host=None):
        """Host (ideally pinned) tensors in and out; copies and a stream wait happen inside the call."""
        def hp(t):
            if t is None:
                return None
            assert (not t.is_cuda) and t.is_contiguous()
            return C.c_void_p(t.data_ptr())
        self._check(self.lib.dsmoe_moe_forward_host(self.h, layer, hp(x_host), hp(logits_host), n_tokens, hp(out_host),
                                                    hp(selected_host), hp(weights_host)))

    def moe_forward_host_async(self, layer: int, x_host, logits_host, n_tokens: int, out_host, selected_host=None,
                               weights_host=None):
        """The same, queued on the handle's stream without waiting (pinned host tensors only); ``host_synchronize``
        waits. One call in flight per handle; two handles used in turn overlap copies with kernels."""
        def hp(t):
            if t is None:
                return None
            assert (not t.is_cuda) and t.is_contiguous() and t.is_pinned()
            return C.c_void_p(t.data_ptr())
        self._check(self.lib.dsmoe_moe_forward_host_async(self.h, layer, hp(x_host), hp(logits_host), n_tokens,
                                                          hp(out_host), hp(selected_host), hp(weights_host)))

    def host_synchronize(self):
        self._check(self.lib.dsmoe_host_synchronize(self.h))


class MoeLayer:
    """One layer's routed experts resident on the device, with the upload-time re-layout applied.

    Counterpart of the expert-tensor upload (engine/src/engine.rs:77-90) plus step "h" of
    Session::decode_attn_out_and_ffn (engine/src/session.rs:1989-2155)."""

    def __init__(self, kernels: MoeKernels, gate_bytes, up_bytes, down_bytes, layout: int = LAYOUT_ROWSOA,
                 layer: int = 0):
        self.k = kernels
        cfg = kernels.cfg
        dev = torch.device("cuda", kernels.device)
        self.xq_blocks, self.mid_blocks = cfg.n_embd // QK_K, cfg.n_ff // QK_K
        as_dev = lambda a: (a if isinstance(a, torch.Tensor) else torch.from_numpy(a)).to(dev).contiguous().view(-1)
        gate, up, down = as_dev(gate_bytes), as_dev(up_bytes), as_dev(down_bytes)
        assert gate.numel() == cfg.n_expert * cfg.n_ff * self.xq_blocks * IQ2XXS_BYTES
        assert down.numel() == cfg.n_expert * cfg.n_embd * self.mid_blocks * Q2K_BYTES
        if layout == LAYOUT_ROWSOA:
            g2, u2, d2 = torch.empty_like(gate), torch.empty_like(up), torch.empty_like(down)
            kernels.relayout_iq2xxs(gate, g2, cfg.n_expert * cfg.n_ff, self.xq_blocks)
            kernels.relayout_iq2xxs(up, u2, cfg.n_expert * cfg.n_ff, self.xq_blocks)
            kernels.relayout_q2k(down, d2, cfg.n_expert * cfg.n_embd, self.mid_blocks)
            torch.cuda.synchronize()
            gate, up, down = g2, u2, d2
        self.gate, self.up, self.down, self.layout, self.layer = gate, up, down, layout, layer
        kernels.layer_register(layer, gate, up, down, layout)

    @property
    def packed_bytes_per_expert(self) -> int:
        c = self.k.cfg
        return 2 * c.n_ff * self.xq_blocks * IQ2XXS_BYTES + c.n_embd * self.mid_blocks * Q2K_BYTES

    def forward(self, x, logits, out=None, selected_out=None, weights_out=None):
        n = x.shape[0]
        if out is None:
            out = torch.empty((n, self.k.cfg.n_embd), dtype=torch.float32, device=x.device)
        self.k.moe_forward(self.layer, x, logits, n, out, selected_out, weights_out)
        return out


def q8k_empty(n_rows: int, blocks: int, device) -> torch.Tensor:
    return torch.empty((n_rows, blocks, Q8K_BYTES), dtype=torch.uint8, device=device)
