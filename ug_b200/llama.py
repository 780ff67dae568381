"""Host-side mirror of ug-llama's model API over the fused Llama engine.

``Config`` and ``Model`` follow ug-llama/src/model.rs:10-30,298-374: the same
field names, the same safetensors weight names, ``Model.new`` / ``Model.fwd``.
``fwd`` takes one new token per sequence (the graph-replayed decode step) or a
block of them (the causal prefill path); the KV cache that the reference
threads through ``fwd`` as ``&mut [Cache]`` lives inside the engine.  Weights
come from host arrays (``Model.new``) or from .safetensors files
(``Model.from_safetensors``); ``tp=(rank, size)`` builds the tensor-parallel variant.
"""
import ctypes as C

import numpy as np

from ._lib import lib
from .device import DType, UgError
from .llama_config import Config, weight_names, weight_shape  # noqa: F401 (re-exported)


class _CConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("hidden", "layers", "n_heads", "n_kv_heads", "head_dim", "ffn",
                                          "vocab", "max_pos")] + \
               [("rope_theta", C.c_float), ("rms_eps", C.c_float), ("rope_interleaved", C.c_int32)]


class Model:
    """Model::new / Model::fwd for seq_len == 1 over ``batch`` independent sequences."""

    def __init__(self, cfg, dev, batch, t_max, tp=None):
        """``tp = (rank, size)`` builds the tensor-parallel variant: this process keeps rank's share of
        heads, FFN columns and vocabulary; call :meth:`connect` on every rank before the first step."""
        if not cfg.tie_word_embeddings:
            raise UgError(6, "tie_word_embeddings == false is not supported yet")   # model.rs:318
        self.cfg, self.dev, self.batch = cfg, dev, batch
        self.tp = tp
        cc = _CConfig(cfg.hidden_size, cfg.num_hidden_layers, cfg.num_attention_heads,
                      cfg.num_key_value_heads, cfg.head_dim(), cfg.intermediate_size, cfg.vocab_size,
                      cfg.max_position_embeddings, cfg.rope_theta, cfg.rms_norm_eps,
                      int(cfg.rope_interleaved))
        h = C.c_void_p()
        if tp is None:
            dev._check(lib.ugb_llama_create(dev._h, C.byref(cc), batch, t_max, C.byref(h)))
        else:
            dev._check(lib.ugb_llama_create_tp(dev._h, C.byref(cc), batch, t_max, tp[0], tp[1], C.byref(h)))
        self._h = h
        info = [C.c_int32() for _ in range(5)]
        lib.ugb_llama_tp_info(h, *[C.byref(i) for i in info])
        self.tp_rank, self.tp_size, self.vocab_local, self.vocab_offset, self.kv_heads_local = (i.value for i in info)

    @classmethod
    def new(cls, cfg, weights, dev, batch, t_max, tp=None, group=None):
        """``weights``: name -> host array; uint16 arrays are bf16 bit patterns, float32 arrays
        are norm weights (or matrices to be rounded to bf16 on the device).  Tensor parallel
        (``tp``): every rank passes the whole tensors and ``group`` (ug_b200.dist.Group)."""
        m = cls(cfg, dev, batch, t_max, tp=tp)
        for name in weight_names(cfg):
            m.load_weight(name, weights[name])
        if tp is not None:
            m.connect(group)
        return m

    @classmethod
    def from_safetensors(cls, cfg, st, dev, batch, t_max, tp=None, group=None):
        """Model::new (model.rs:298-363) from a ``ug_b200.safetensors.MmapedSafetensors``: projection and
        embedding matrices keep their stored BF16 / F32 (F16 goes through F32), norm weights are cast to F32."""
        from .device import DType
        m = cls(cfg, dev, batch, t_max, tp=tp)
        for name in weight_names(cfg):
            src_dtype, shape = st.get(name)
            if len(shape) == 1 or src_dtype not in (DType.BF16, DType.F32):
                _, s = st.load_slice_with_cast(name, DType.F32, dev)
            else:
                _, s = st.load_slice(name, dev)
            dev._check(lib.ugb_llama_load_weight(m._h, name.encode(), s._h))
            dev.synchronize()
        if tp is not None:
            m.connect(group)
        return m

    def connect(self, group):
        """Maps the peers' exchange blocks (collective over ``group``; no-op for one rank)."""
        if self.tp is None or self.tp_size == 1:
            return
        buf = C.create_string_buffer(64)
        self.dev._check(lib.ugb_llama_tp_export(self._h, buf, 64))
        handles = b"".join(group.all_gather_bytes(buf.raw))
        self.dev._check(lib.ugb_llama_tp_connect(self._h, handles, 64, self.tp_size))
        self.dev.synchronize()
        group.barrier()          # nobody steps before everybody has mapped everybody

    def load_weight(self, name, arr):
        arr = np.ascontiguousarray(arr)
        s = self.dev.slice_from_values(arr.ravel(), bf16=(arr.dtype == np.uint16))
        self.dev._check(lib.ugb_llama_load_weight(self._h, name.encode(), s._h))
        self.dev.synchronize()

    def close(self):
        h, self._h = self._h, None
        if h:
            lib.ugb_llama_destroy(h)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_option(self, key, value):
        self.dev._check(lib.ugb_llama_set_option(self._h, key.encode(), value))

    def reset(self, pos=0):
        self.dev._check(lib.ugb_llama_reset(self._h, pos))

    @property
    def position(self):
        return lib.ugb_llama_position(self._h)

    def fwd(self, tokens):
        """Model::fwd on explicit token ids, asynchronous: int32 [batch] or [batch, 1] is one
        decode step; [batch, t] with t > 1 appends t positions (causal prefill) and keeps the
        logits of every position for :meth:`prefill_logits`."""
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        if tokens.ndim == 2 and tokens.shape[1] > 1:
            return self.prefill(tokens, all_logits=True)
        s = self.dev.slice_from_values(tokens.reshape(-1))
        self.dev._check(lib.ugb_llama_decode(self._h, s._h, 1))

    def prefill(self, tokens, all_logits=False):
        """Appends ``tokens`` (int32 [batch, t], host array or device Slice of batch*t ids) to
        every sequence; :meth:`logits` / :meth:`next_tokens` then refer to the last position."""
        if isinstance(tokens, np.ndarray) or not hasattr(tokens, "_h"):
            tokens = np.ascontiguousarray(tokens, dtype=np.int32)
            if tokens.ndim != 2 or tokens.shape[0] != self.batch:
                raise UgError(4, f"prefill tokens must be [batch={self.batch}, t], got {tokens.shape}")
            t = tokens.shape[1]
            s = self.dev.slice_from_values(tokens.reshape(-1))
        else:
            s, t = tokens, tokens.len // self.batch
        self.dev._check(lib.ugb_llama_prefill(self._h, s._h, t, int(all_logits)))
        self._prefill_t = t if all_logits else getattr(self, "_prefill_t", 0)

    def prefill_logits(self):
        """f32 [batch, t, vocab] of the last ``all_logits`` prefill (what Model::fwd returns)."""
        t = getattr(self, "_prefill_t", 0)
        out = np.empty((self.batch, t, self.vocab_local), np.float32)
        self.dev._check(lib.ugb_llama_read(self._h, 3, out.ctypes.data, out.size))
        return out

    def decode(self, n_steps):
        """Greedy decoding: each step feeds the previous step's argmax; asynchronous."""
        self.dev._check(lib.ugb_llama_decode(self._h, None, n_steps))

    def logits(self):
        """f32 [batch, vocab]; a tensor-parallel rank returns its columns
        [vocab_offset, vocab_offset + vocab_local)."""
        out = np.empty((self.batch, self.vocab_local), np.float32)
        self.dev._check(lib.ugb_llama_read(self._h, 0, out.ctypes.data, out.size))
        return out

    def next_tokens(self):
        out = np.empty(self.batch, np.int32)
        self.dev._check(lib.ugb_llama_read(self._h, 1, out.ctypes.data, out.size))
        return out

    def hidden(self):
        out = np.empty((self.batch, self.cfg.hidden_size), np.float32)
        self.dev._check(lib.ugb_llama_read(self._h, 2, out.ctypes.data, out.size))
        return out

    def kv_cache(self, layer, which):
        """bf16 bit patterns [batch, n_kv_heads, kv_positions, head_dim] of K (0) or V (1)."""
        t = lib.ugb_llama_kv_positions(self._h)
        out = np.empty((self.batch, self.kv_heads_local, t, self.cfg.head_dim()), np.uint16)
        self.dev._check(lib.ugb_llama_read_kv(self._h, layer, which, out.ctypes.data, out.size))
        return out

    KERNELS = {"qkv_gemm": 0, "decode_attention": 1, "o_gemm": 2, "gate_up_gemm": 3, "down_gemm": 4,
               "lm_head_gemm": 5}

    def time_kernel(self, name, iters=20):
        """Milliseconds one decode step spends in kernel type ``name`` (all layers), CUDA events."""
        ms = C.c_float()
        self.dev._check(lib.ugb_llama_time_kernel(self._h, self.KERNELS[name], iters, C.byref(ms)))
        return ms.value
