"""Host side of the Q8_0 Llama forward: the structs of bench/bpd_cpu.c:5537-5588 of the reference
(bpd_llama_config, bpd_llama_layer_weights, bpd_llama_weights) filled with device pointers, and the
call sequence of its C-loop wrapper (inference/llamatov_c_inference.py:62-78): prefill once, then one
token per step against the f16 KV cache.

``SyntheticLlama`` makes a random model of a given shape on the host (Q8_0 matrices, norm weights);
``DeviceLlama`` uploads one and runs ``bpd_llama_forward_cuda`` on it.  There is no CPU path here.
"""
import ctypes as C

import numpy as np

from . import capi, synth

LAYER_FIELDS = ("attn_norm_w", "w_q", "w_k", "w_v", "w_o", "ffn_norm_w", "w_gate", "w_up", "w_down")


def make_config(n_layers, n_heads, n_kv_heads, head_dim, ffn_dim, vocab_size, max_seq_len, rms_eps=1e-5, rope_base=500000.0,
                rope_dim=None, kv_cache_f16=1):
    return capi.LlamaConfig(n_layers, n_heads, n_kv_heads, head_dim, n_heads * head_dim, ffn_dim, vocab_size, max_seq_len,
                            rms_eps, rope_base, head_dim if rope_dim is None else rope_dim, kv_cache_f16)


class SyntheticLlama:
    """Random Q8_0 model on the host.  Block scales are chosen so that a weight row has unit norm on
    average: projections then keep activations O(1) and attention scores O(1), i.e. the softmax is not
    saturated and small numerical differences stay small."""

    def __init__(self, cfg, seed=0, rope_freqs=True):
        self.cfg = cfg
        rng = np.random.default_rng(seed)
        E, F, D = cfg.embed_dim, cfg.ffn_dim, cfg.head_dim
        kv = cfg.n_kv_heads * D

        def mat(rows, cols):
            return synth.q8_0_matrix(rows, cols, rng, scale_sigma=1.0 / (73.0 * np.sqrt(cols)))

        def norm():
            return (1.0 + 0.1 * rng.standard_normal(E)).astype(np.float32)

        self.token_embd = synth.q8_0_matrix(cfg.vocab_size, E, rng, scale_sigma=1.0 / 73.0)
        self.layers = []
        for _ in range(cfg.n_layers):
            self.layers.append(dict(attn_norm_w=norm(), w_q=mat(E, E), w_k=mat(kv, E), w_v=mat(kv, E), w_o=mat(E, E),
                                    ffn_norm_w=norm(), w_gate=mat(F, E), w_up=mat(F, E), w_down=mat(E, F)))
        self.output_norm_w = norm()
        self.output_w = mat(cfg.vocab_size, E)
        self.rope_freqs = ((1.0 + rng.random(cfg.rope_dim // 2) * 3.0).astype(np.float32) if rope_freqs else None)

    def weight_bytes(self):
        n = self.token_embd.nbytes + self.output_w.nbytes
        return n + sum(sum(v.nbytes for v in layer.values()) for layer in self.layers)

    def kv_cache(self):
        """Zeroed K and V caches [n_layers][max_seq_len][n_kv_heads*head_dim] of the configured type."""
        c = self.cfg
        shape = (c.n_layers, c.max_seq_len, c.n_kv_heads * c.head_dim)
        dt = np.uint16 if c.kv_cache_f16 else np.float32
        return np.zeros(shape, dt), np.zeros(shape, dt)

    def host_structs(self):
        """(LlamaWeights, keep-alive list) with pointers into this object's numpy arrays: the argument of
        the CPU checker and of the compiled reference."""
        layers = (capi.LlamaLayerWeights * max(1, len(self.layers)))()
        for i, layer in enumerate(self.layers):
            for f in LAYER_FIELDS:
                setattr(layers[i], f, layer[f].ctypes.data)
        w = capi.LlamaWeights(self.token_embd.ctypes.data, layers, self.output_norm_w.ctypes.data,
                              self.output_w.ctypes.data, self.rope_freqs.ctypes.data if self.rope_freqs is not None else None)
        return w, [layers]


class DeviceLlama:
    """A SyntheticLlama resident on the device, with its KV caches."""

    def __init__(self, model, lib=None):
        self.lib = lib = lib or capi.load()
        self.model, self.cfg = model, model.cfg
        self._allocs = []
        self.layers = (capi.LlamaLayerWeights * max(1, len(model.layers)))()
        for i, layer in enumerate(model.layers):
            for f in LAYER_FIELDS:
                setattr(self.layers[i], f, self._up(layer[f]))
        self.weights = capi.LlamaWeights(self._up(model.token_embd), self.layers, self._up(model.output_norm_w),
                                         self._up(model.output_w),
                                         self._up(model.rope_freqs) if model.rope_freqs is not None else None)
        k, v = model.kv_cache()
        self.kv_bytes = k.nbytes
        self.d_k, self.d_v = self._up(k), self._up(v)
        self.stream = lib.bpdq_stream_create()
        capi.check(lib.bpdq_last_status(), "DeviceLlama setup")

    def _up(self, arr):
        arr = np.ascontiguousarray(arr)
        p = self.lib.bpdq_alloc(max(arr.nbytes, 16))
        self.lib.bpdq_h2d(p, arr.ctypes.data, arr.nbytes)
        self._allocs.append(p)
        return p

    def retile(self):
        """Makes the re-tiled copy of every Q8_0 matrix (device-side permutation); prefills then run each
        product once over the weights on the tensor cores.  Costs a second copy of the matrices."""
        lib, c = self.lib, self.cfg
        E, F, kv = c.embed_dim, c.ffn_dim, c.n_kv_heads * c.head_dim
        shapes = dict(w_q=(E, E), w_k=(kv, E), w_v=(kv, E), w_o=(E, E), w_gate=(F, E), w_up=(F, E), w_down=(E, F))

        def tile(ptr, rows, cols):
            t = lib.bpdq_alloc(lib.bpd_q8_0_tiles_bytes(rows, cols))
            capi.check(lib.bpd_repack_q8_0_tiles_cuda(ptr, t, rows, cols, self.stream), "bpd_repack_q8_0_tiles_cuda")
            self._allocs.append(t)
            return t

        self.tile_layers = (capi.LlamaLayerWeights * max(1, len(self.model.layers)))()
        for i in range(len(self.model.layers)):
            for f, (rows, cols) in shapes.items():
                setattr(self.tile_layers[i], f, tile(getattr(self.layers[i], f), rows, cols))
        self.tiles = capi.LlamaWeights(None, self.tile_layers, None, tile(self.weights.output_w, c.vocab_size, E), None)
        capi.check(lib.bpdq_stream_sync(self.stream))

    def reset_cache(self):
        capi.check(self.lib.bpdq_memset_async(self.d_k, 0, self.kv_bytes, self.stream))
        capi.check(self.lib.bpdq_memset_async(self.d_v, 0, self.kv_bytes, self.stream))

    def forward(self, token_ids, pos_ids, kv_pos):
        """Runs the tokens through all layers; returns (logits [n, vocab], argmax tokens [n])."""
        lib = self.lib
        token_ids = np.ascontiguousarray(token_ids, np.int32)
        pos_ids = np.ascontiguousarray(pos_ids, np.int32)
        n = token_ids.size
        d_tok, d_pos = lib.bpdq_alloc(max(16, 4 * n)), lib.bpdq_alloc(max(16, 4 * n))
        d_logits, d_out = lib.bpdq_alloc(4 * n * self.cfg.vocab_size), lib.bpdq_alloc(8 * n)
        try:
            lib.bpdq_h2d(d_tok, token_ids.ctypes.data, 4 * n)
            lib.bpdq_h2d(d_pos, pos_ids.ctypes.data, 4 * n)
            tiles = C.byref(self.tiles) if getattr(self, "tiles", None) is not None else None
            capi.check(lib.bpd_llama_forward_tiles_cuda(d_tok, n, C.byref(self.weights), tiles, C.byref(self.cfg), d_pos, kv_pos,
                                                        self.d_k, self.d_v, d_logits, d_out, self.stream),
                       "bpd_llama_forward_tiles_cuda")
            capi.check(lib.bpdq_stream_sync(self.stream))
            logits = np.empty((n, self.cfg.vocab_size), np.float32)
            tokens = np.empty(n, np.int64)
            lib.bpdq_d2h(logits.ctypes.data, d_logits, logits.nbytes)
            lib.bpdq_d2h(tokens.ctypes.data, d_out, tokens.nbytes)
            capi.check(lib.bpdq_last_status(), "llama forward")
            return logits, tokens
        finally:
            for p in (d_tok, d_pos, d_logits, d_out):
                lib.bpdq_free(p)

    def read_cache(self):
        k, v = self.model.kv_cache()
        self.lib.bpdq_stream_sync(self.stream)
        self.lib.bpdq_d2h(k.ctypes.data, self.d_k, k.nbytes)
        self.lib.bpdq_d2h(v.ctypes.data, self.d_v, v.nbytes)
        return k, v

    def close(self):
        self.lib.bpdq_stream_sync(self.stream)
        for p in self._allocs:
            self.lib.bpdq_free(p)
        self._allocs = []
        self.lib.bpdq_stream_destroy(self.stream)
