"""Input generators shared by ``make_golden.py`` and the tests.

The formula fixtures restate the generators of the reference's own tests
(tests/core/backend/test_quantized_linear_backend.cpp:89-169,
tests/core/backend/test_nn_backend.cpp:2079-2216); the seeded cases follow the
baseline configurations (shapes and value distributions) at sizes the CPU
checkers finish in seconds.
"""
from __future__ import annotations

import numpy as np

SEED = 20241


# ---- fixtures by formula (the reference tests' generators, restated) -----------------

def aligned_weight() -> np.ndarray:
    v = np.array([((i % 19) - 9) * np.float32(0.1375) for i in range(3 * 32)], np.float32)
    v[0], v[31], v[32], v[-1] = -2.0, 1.75, 3.0, -4.0
    return v.reshape(3, 32)


def aligned_input() -> np.ndarray:
    return np.array([((i % 11) - 5) * np.float32(0.2) for i in range(2 * 32)], np.float32).reshape(2, 32)


def aligned_upstream() -> np.ndarray:
    return np.array([0.25, -0.75, 1.5, -1.0, 0.5, 0.125], np.float32).reshape(2, 3)


def edge_weight() -> np.ndarray:
    n = 33
    v = np.array([((i % 37) - 18) * np.float32(0.0625) for i in range(n * n)], np.float32)
    v[0], v[31], v[32], v[1023], v[1024], v[-1] = -3.0, 2.5, -2.75, 4.0, -4.5, 5.0
    return v.reshape(n, n)


def edge_input() -> np.ndarray:
    return np.array([((i % 17) - 8) * np.float32(0.125) for i in range(2 * 33)], np.float32).reshape(2, 33)


def edge_upstream() -> np.ndarray:
    return np.array([((i % 13) - 6) * np.float32(0.075) for i in range(2 * 33)], np.float32).reshape(2, 33)


def paged_fixture():
    heads, time, width, block_size, physical = 2, 5, 3, 2, 5
    table = np.array([3, 0, 4], np.uint32)
    n = heads * time * width
    qv = np.array([((i % 7) - 3) * np.float32(0.17) for i in range(n)], np.float32).reshape(1, heads, time, width)
    kv = np.array([((i % 5) - 2) * np.float32(0.23) for i in range(n)], np.float32).reshape(1, heads, time, width)
    vv = np.array([((i % 11) - 5) * np.float32(0.11) for i in range(n)], np.float32).reshape(1, heads, time, width)
    key_pages = np.full((physical, heads, block_size, width), -777.0, np.float32)
    value_pages = np.full((physical, heads, block_size, width), 777.0, np.float32)
    for h in range(heads):
        for p in range(time):
            key_pages[table[p // block_size], h, p % block_size] = kv[0, h, p]
            value_pages[table[p // block_size], h, p % block_size] = vv[0, h, p]
    query = qv[0, :, time - 1, :].copy()
    return qv, kv, vv, query, key_pages, value_pages, table, time



def seeded_cases():
    """Returns the seeded random inputs in the order the generator draws them."""
    rng = np.random.default_rng(SEED)
    W1 = (rng.standard_normal((1024, 512)) * 0.02).astype(np.float32)
    X1 = rng.standard_normal((64, 512)).astype(np.float32)
    dY1 = (rng.standard_normal((4, 1024)) * 0.01).astype(np.float32)
    H, d, bs, P, n = 8, 128, 16, 24, 301
    q = rng.standard_normal((1, 32, d)).astype(np.float32)
    K = rng.standard_normal((P, H, bs, d)).astype(np.float32)
    V = rng.standard_normal((P, H, bs, d)).astype(np.float32)
    tab = rng.permutation(P)[: -(-n // bs)].astype(np.uint32)
    return dict(W1=W1, X1=X1, dY1=dY1, q=q, K=K, V=V, table=tab, seq_len=n)


ROPE_POSITIONS = (0, 15, 16, 301, 2048)


def decode_glue_inputs() -> dict:
    """Seeded inputs of the decode-step primitives (RMSNorm, split-half RoPE, SiLU / SwiGLU hidden
    state, greedy choice, token-by-token paged cache), including the special values the reference
    treats explicitly: silu(-inf) = -0.0, large magnitudes on both sigmoid branches, ties and a
    maximum in the last slot for the greedy choice."""
    rng = np.random.default_rng(20250)
    special = np.array([np.inf, -np.inf, 0.0, -0.0, 88.0, -88.0, 100.0, -100.0, -104.0, 1e-30, -1e-30], np.float32)
    gate = np.concatenate([(rng.standard_normal(2037) * 6).astype(np.float32), special])
    greedy = rng.standard_normal((6, 97)).astype(np.float32)
    greedy[1, 40] = greedy[1, 70] = greedy[1].max() + 1.0     # tie: the first index wins
    greedy[2, 96] = greedy[2].max() + 1.0                      # maximum in the last slot
    greedy[3, 0] = greedy[3].max() + 1.0                       # maximum in the first slot
    greedy[4, :] = 0.5                                         # all equal
    return {
        "rms_x": (rng.standard_normal((6, 1024)) * np.array([1, 10, 1e-3, 1e3, 1, 1])[:, None]).astype(np.float32),
        "rms_scale": (1.0 + 0.1 * rng.standard_normal(1024)).astype(np.float32),
        "rope_x": rng.standard_normal((2, 3, 1, 128)).astype(np.float32),
        "silu_gate": gate,
        "silu_up": rng.standard_normal(gate.size).astype(np.float32),
        "greedy_logits": greedy,
        "cache_q": rng.standard_normal((18, 2, 8)).astype(np.float32),
        "cache_k": rng.standard_normal((18, 2, 8)).astype(np.float32),
        "cache_v": rng.standard_normal((18, 2, 8)).astype(np.float32),
    }


def lora_inputs() -> dict:
    """A small Linear with a low-rank adapter: x [5, 96], A [4, 96], B [40, 4], scale = alpha / rank."""
    rng = np.random.default_rng(4040)
    return {"x": rng.standard_normal((5, 96)).astype(np.float32),
            "a": (rng.standard_normal((4, 96)) * 0.1).astype(np.float32),
            "b": (rng.standard_normal((40, 4)) * 0.1).astype(np.float32),
            "w": (rng.standard_normal((40, 96)) * 0.02).astype(np.float32),
            "scale": np.float32(8.0 / 4.0)}
