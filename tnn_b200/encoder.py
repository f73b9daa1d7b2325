"""Host-side mirror of the fused encoder: packed device weights + the launch sequence of one Forward.

`Encoder.from_workload` does what the fused layers' `Init` does in the TNN plug-in: upload the fp32 `[K,N]` MatMul
weights, pre-pack them to half-precision `[N,K]` (Q/K/V concatenated into one `[3H,H]` operand), keep biases and
LayerNorm parameters in fp32.  `forward` is `Instance::Forward` for the fused graph: fp32 activations in, the fused
region in fp16/bf16, fp32 out.  All compute goes through the C ABI (tnn_b200.capi); there is no torch math here.
"""
import ctypes

import numpy as np
import torch

from . import capi, ops


class Encoder:
    def __init__(self, cfg, dtype, device):
        self.cfg = cfg
        self.dtype = dtype
        self.device = device
        self.layers = []          # dicts of device tensors (kept alive here)
        self._c_layers = None
        self._ws = None
        self._ws_key = None
        self.fold = False

    @classmethod
    def from_workload(cls, wl, dtype=torch.float16, device="cuda", fold_layernorm=False):
        """`fold_layernorm`: prepare the weights for the five-launch form of a layer (both LayerNorms folded into
        the neighbouring GEMMs); only full encoder layers can be folded.  Off by default: at BERT's K = 768 the
        seven-launch layer with its own LayerNorm kernel is the faster one, and it is what the TNN plug-in runs."""
        enc = cls(wl.cfg, dtype, torch.device(device))
        enc.fold = bool(fold_layernorm) and wl.cfg.with_ffn
        H, F = wl.cfg.hidden, wl.cfg.ffn

        def dev(a):
            return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(enc.device)

        prev = None
        for lw in wl.weights:
            L = {}
            w_qkv = torch.empty((3 * H, H), dtype=dtype, device=enc.device)
            L["b_qkv"] = dev(np.concatenate([lw.bq, lw.bk, lw.bv]))
            if enc.fold and prev is not None:
                # LN2 of the previous layer is folded into this layer's QKV projection
                w_cat = dev(np.concatenate([lw.wq, lw.wk, lw.wv], axis=1))
                _, L["qkv_c1"], L["qkv_c2"] = ops.fold_layernorm_weight(w_cat, prev["ln2_g"], prev["ln2_b"],
                                                                        L["b_qkv"], dtype, out=w_qkv)
            else:
                for i, w in enumerate((lw.wq, lw.wk, lw.wv)):
                    ops.pack_weight(dev(w), dtype, out=w_qkv[i * H:(i + 1) * H])
            L["w_qkv"] = w_qkv
            L["w_o"] = ops.pack_weight(dev(lw.wo), dtype)
            L["b_o"] = dev(lw.bo)
            L["ln1_g"], L["ln1_b"] = dev(lw.ln1_g), dev(lw.ln1_b)
            if wl.cfg.with_ffn:
                L["b_ffn1"] = dev(lw.b1)
                if enc.fold:
                    L["w_ffn1"], L["ffn1_c1"], L["ffn1_c2"] = ops.fold_layernorm_weight(
                        dev(lw.w1), L["ln1_g"], L["ln1_b"], L["b_ffn1"], dtype)
                else:
                    L["w_ffn1"] = ops.pack_weight(dev(lw.w1), dtype)
                L["w_ffn2"] = ops.pack_weight(dev(lw.w2), dtype)
                L["b_ffn2"] = dev(lw.b2)
                L["ln2_g"], L["ln2_b"] = dev(lw.ln2_g), dev(lw.ln2_b)
            enc.layers.append(L)
            prev = L
        torch.cuda.synchronize(enc.device)
        return enc

    # ------------------------------------------------------------------ layer-by-layer path (any config)
    def forward_ops(self, x_f32, mask_add=None, out_f32=True):
        """x_f32 `[B,S,H]` fp32 device tensor -> `[B,S,H]`; one launch per fused layer."""
        if self.fold:
            return self._forward_ops_folded(x_f32, mask_add, out_f32)
        cfg = self.cfg
        B, S, H = x_f32.shape
        h = ops.convert(x_f32.contiguous(), self.dtype)
        kv_len = None
        m2 = None
        if mask_add is not None:
            m2 = mask_add.reshape(B, S).contiguous()
            kv_len = ops.mask_to_kv_len(m2)
        for L in self.layers:
            qkv = ops.linear(h, L["w_qkv"], L["b_qkv"])
            ctx = ops.attention(qkv, cfg.heads, m2, kv_len, scale=1.0 / float(np.sqrt(cfg.head_dim)))
            t = ops.linear(ctx, L["w_o"], L["b_o"], residual=h, epilogue=ops.EPI_BIAS_RESIDUAL)
            a = ops.add_layernorm(t, L["ln1_g"], L["ln1_b"], cfg.ln_eps)
            if cfg.with_ffn:
                f1 = ops.linear(a, L["w_ffn1"], L["b_ffn1"], epilogue=ops.EPI_BIAS_GELU)
                t2 = ops.linear(f1, L["w_ffn2"], L["b_ffn2"], residual=a, epilogue=ops.EPI_BIAS_RESIDUAL)
                h = ops.add_layernorm(t2, L["ln2_g"], L["ln2_b"], cfg.ln_eps)
            else:
                h = a
        return ops.convert(h, torch.float32) if out_f32 else h

    def _forward_ops_folded(self, x_f32, mask_add, out_f32):
        """The five-launch layer, one C-ABI call per launch (what b200_encoder_fwd does with fold_layernorm = 1)."""
        cfg = self.cfg
        B, S, H = x_f32.shape
        eps = cfg.ln_eps
        h0 = ops.convert(x_f32.contiguous(), self.dtype)
        m2 = kv_len = None
        if mask_add is not None:
            m2 = mask_add.reshape(B, S).contiguous()
            kv_len = ops.mask_to_kv_len(m2)
        st1 = ops.stats_buffer(B * S, H, x_f32.device)
        st2 = ops.stats_buffer(B * S, H, x_f32.device)
        t2 = None
        prev = None
        for L in self.layers:
            if prev is None:
                qkv = ops.linear(h0, L["w_qkv"], L["b_qkv"])
            else:
                qkv = ops.linear(t2, L["w_qkv"], None, ln_in=(st2, L["qkv_c1"], L["qkv_c2"]), ln_eps=eps)
            ctx = ops.attention(qkv, cfg.heads, m2, kv_len, scale=1.0 / float(np.sqrt(cfg.head_dim)))
            if prev is None:
                t1 = ops.linear(ctx, L["w_o"], L["b_o"], residual=h0, epilogue=ops.EPI_BIAS_RESIDUAL,
                                out_stats=st1, ln_eps=eps)
            else:
                t1 = ops.linear(ctx, L["w_o"], L["b_o"], residual=t2, epilogue=ops.EPI_BIAS_RESIDUAL,
                                out_stats=st1, res_ln=(st2, prev["ln2_g"], prev["ln2_b"]), ln_eps=eps)
            f1 = ops.linear(t1, L["w_ffn1"], None, epilogue=ops.EPI_BIAS_GELU,
                            ln_in=(st1, L["ffn1_c1"], L["ffn1_c2"]), ln_eps=eps)
            t2 = ops.linear(f1, L["w_ffn2"], L["b_ffn2"], residual=t1, epilogue=ops.EPI_BIAS_RESIDUAL,
                            out_stats=st2, res_ln=(st1, L["ln1_g"], L["ln1_b"]), ln_eps=eps)
            prev = L
        h = ops.add_layernorm(t2, prev["ln2_g"], prev["ln2_b"], eps)
        return ops.convert(h, torch.float32) if out_f32 else h

    # ------------------------------------------------------------------ single-call path (full encoder layers)
    def _layer_array(self):
        if self._c_layers is None:
            arr = (capi.EncoderLayerWeights * len(self.layers))()
            for i, L in enumerate(self.layers):
                c = arr[i]
                c.w_qkv, c.b_qkv = L["w_qkv"].data_ptr(), L["b_qkv"].data_ptr()
                c.w_o, c.b_o = L["w_o"].data_ptr(), L["b_o"].data_ptr()
                c.ln1_gamma, c.ln1_beta = L["ln1_g"].data_ptr(), L["ln1_b"].data_ptr()
                c.w_ffn1, c.b_ffn1 = L["w_ffn1"].data_ptr(), L["b_ffn1"].data_ptr()
                c.w_ffn2, c.b_ffn2 = L["w_ffn2"].data_ptr(), L["b_ffn2"].data_ptr()
                c.ln2_gamma, c.ln2_beta = L["ln2_g"].data_ptr(), L["ln2_b"].data_ptr()
                if self.fold:
                    c.ffn1_c1, c.ffn1_c2 = L["ffn1_c1"].data_ptr(), L["ffn1_c2"].data_ptr()
                    if "qkv_c1" in L:
                        c.qkv_c1, c.qkv_c2 = L["qkv_c1"].data_ptr(), L["qkv_c2"].data_ptr()
            self._c_layers = arr
        return self._c_layers

    def workspace(self, tokens):
        key = tokens
        if self._ws_key != key:
            n = capi.lib().b200_encoder_workspace_bytes(tokens, self.cfg.hidden, self.cfg.ffn,
                                                        capi.dtype_code(self.dtype))
            self._ws = torch.empty((n + 256,), dtype=torch.uint8, device=self.device)
            self._ws_key = key
        off = (-self._ws.data_ptr()) % 256
        return self._ws.data_ptr() + off

    def forward_hidden(self, hidden, mask2d=None, kv_len=None):
        """In-place stack over `hidden` `[B,S,H]` (fp16/bf16 device tensor) through b200_encoder_fwd."""
        if not self.cfg.with_ffn:
            raise ValueError("b200_encoder_fwd runs full encoder layers; use forward_ops for attention-only blocks")
        B, S, H = hidden.shape
        d = capi.EncoderDesc()
        d.hidden = hidden.data_ptr()
        d.mask_add = capi.ptr(mask2d)
        d.kv_len = capi.ptr(kv_len)
        d.layers = self._layer_array()
        d.workspace = self.workspace(B * S)
        d.B, d.S, d.H, d.F = B, S, H, self.cfg.ffn
        d.heads, d.num_layers = self.cfg.heads, len(self.layers)
        d.dtype = capi.dtype_code(self.dtype)
        d.ln_eps = float(self.cfg.ln_eps)
        d.mask_exclude_below = -5000.0
        d.fold_layernorm = 1 if self.fold else 0
        rc = capi.lib().b200_encoder_fwd(ctypes.byref(d), capi.stream_ptr())
        capi.check(rc, "b200_encoder_fwd")
        return hidden

    def forward(self, x_f32, mask_add=None):
        """fp32 `[B,S,H]` in -> fp32 `[B,S,H]` out (conversion kernels at both ends, as the fused TNN graph does)."""
        if not self.cfg.with_ffn:
            return self.forward_ops(x_f32, mask_add)
        B, S, H = x_f32.shape
        h = ops.convert(x_f32.contiguous(), self.dtype)
        m2 = kv = None
        if mask_add is not None:
            m2 = mask_add.reshape(B, S).contiguous()
            kv = ops.mask_to_kv_len(m2)
        self.forward_hidden(h, m2, kv)
        return ops.convert(h, torch.float32)
