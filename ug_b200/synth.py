"""Seeded synthetic inputs for the benchmark configurations.

A counter-based generator (Philox) with fixed seeds, evaluated on the host so
that the CPU oracle and the GPU see identical bits.  These inputs stand in for
the softmax sweeps and the real checkpoints the reference's own benchmarks
use (ug-cuda/examples/benchmark.rs:77, ug-llama/src/main.rs:105-122), which
are not available offline.
"""
import numpy as np


def rng(seed):
    return np.random.Generator(np.random.Philox(seed))


def normal(seed, shape, std=1.0):
    return (rng(seed).standard_normal(shape, dtype=np.float32) * np.float32(std)).astype(np.float32)


def uniform(seed, shape, lo, hi):
    return rng(seed).uniform(lo, hi, shape).astype(np.float32)


def tokens(seed, shape, vocab):
    return rng(seed).integers(0, vocab, shape, dtype=np.int32)


def to_bf16_bits(x):
    """f32 -> bf16 bit patterns (uint16), round to nearest even."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32)
    # 32-bit wrap-around can only touch NaN bit patterns, which are handled separately below
    rounded = ((u + (np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1)))) >> np.uint32(16)).astype(np.uint16)
    nan = np.isnan(x)
    if nan.any():
        rounded[nan] = ((u[nan] >> np.uint32(16)) | np.uint32(0x40)).astype(np.uint16)
    return rounded


def bf16_bits_to_f32(b):
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def softmax_c1():
    """Config 1: x f32 [1024, 4096] ~ N(0, sigma=2), seed 0."""
    return normal(0, (1024, 4096), 2.0)


def rms_silu_c2(n_rows=8192, n_cols=4096):
    """Config 2: x, gate ~ N(0,1) seeds 1,2; w ~ U(0.5,1.5) seed 3; eps 1e-5."""
    return (normal(1, (n_rows, n_cols)), normal(2, (n_rows, n_cols)),
            uniform(3, (n_cols,), 0.5, 1.5), 1e-5)


def llama_weights(cfg, seed_base=100):
    """Random-init weights of a Llama-shaped model: every matrix ~ N(0, 0.02) rounded to bf16
    (returned as uint16 bit patterns), seed = seed_base + index of the tensor in load order;
    norm weights are ones (f32), the usual initialisation."""
    import os
    from concurrent.futures import ThreadPoolExecutor

    from .llama_config import weight_names, weight_shape

    def one(item):
        i, name = item
        shape = weight_shape(cfg, name)
        if len(shape) == 1:
            return name, np.ones(shape, np.float32)
        return name, to_bf16_bits(normal(seed_base + i, shape, 0.02))

    # every tensor has its own seed, so generating them on several threads changes nothing
    with ThreadPoolExecutor(max_workers=min(16, os.cpu_count() or 1)) as ex:
        return dict(ex.map(one, enumerate(weight_names(cfg))))


def llama_weights_f32(weights):
    """The f32 view of bf16 weights that load_with_cast BF16 -> F32 produces."""
    return {k: (bf16_bits_to_f32(v) if v.dtype == np.uint16 else v) for k, v in weights.items()}
