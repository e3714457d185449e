"""Generate the committed golden fixtures from the reference's own CPU code.

Run where a checkout of quangng2000/riftco-transformer is available (it builds
``oracle/_ref/libriftco_ref.so`` from the reference sources):

    python tests/golden/make_golden.py

Inputs are rebuilt from the index formulas of the reference's own tests
(tests/core/test_quantization.cpp:61-214,
tests/core/backend/test_quantized_linear_backend.cpp:89-169,
tests/core/backend/test_nn_backend.cpp:2079-2216) or from seeded numpy
generators; every output stored here was produced by the reference library,
not by this repository's restatement. The tests compare the restatement (and,
on a GPU, the CUDA path) with these files.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(Path(__file__).resolve().parent))

import oracle  # noqa: E402

OUT = Path(__file__).resolve().parent


def payload_arrays(prefix: str, w: oracle.Nf4Weight) -> dict:
    d = {
        f"{prefix}_codes": w.codes,
        f"{prefix}_shape": np.array([w.out_features, w.in_features, w.block_size, w.scale_block_size], np.int64),
        f"{prefix}_offset": np.array([w.offset], np.float32),
    }
    if w.fp32_scales is not None:
        d[f"{prefix}_fp32_scales"] = w.fp32_scales
    else:
        d[f"{prefix}_scale_codes"] = w.scale_codes
        d[f"{prefix}_second_level"] = w.second_level
    return d


from cases import (ROPE_POSITIONS, aligned_input, aligned_upstream, aligned_weight,  # noqa: E402
                   decode_glue_inputs, edge_input, edge_upstream, edge_weight, lora_inputs, paged_fixture,
                   seeded_cases)


def main() -> None:
    ref = oracle.ref()
    out: dict[str, np.ndarray] = {}

    # -- quantisation known-answer tests ------------------------------------------
    cb = ref.codebook()
    out["codebook"] = cb
    kat = ref.quantize_nf4(cb.reshape(1, 16), 32)
    out.update(payload_arrays("kat_codebook", kat))
    out["kat_codebook_dequant"] = ref.dequantize(kat)

    mid = np.zeros(32, np.float32)
    mid[0] = cb[8] * np.float32(0.5)
    mid[-1] = 1.0
    out["tie_values"] = mid
    out.update(payload_arrays("tie", ref.quantize_nf4(mid.reshape(1, 32), 32)))

    out.update(payload_arrays("zeros33", ref.quantize_nf4(np.zeros((1, 33), np.float32), 32)))

    part = np.full(33, 0.25, np.float32)
    part[0], part[-1] = -2.0, 10.0
    out["partial_values"] = part
    pw = ref.quantize_nf4(part.reshape(1, 33), 32)
    out.update(payload_arrays("partial", pw))
    out["partial_dequant"] = ref.dequantize(pw)

    dq_values = np.repeat(np.arange(33, dtype=np.float32), 32)
    out["dq33_values"] = dq_values
    dq = ref.quantize_nf4_double_quantized(dq_values.reshape(1, -1), 32, 32)
    out.update(payload_arrays("dq33", dq))
    out["dq33_dequant"] = ref.dequantize(dq)

    # nearest-code sweep including exact midpoints
    probes = np.concatenate([np.linspace(-1.25, 1.25, 2001, dtype=np.float32),
                             ((cb[:-1] + cb[1:]) * np.float32(0.5)).astype(np.float32)])
    out["nearest_probes"] = probes
    out["nearest_codes"] = np.array([ref.nearest_code(float(v)) for v in probes], np.uint8)

    # -- linear fixtures of the reference backend test ----------------------------
    for name, W, X, dY in (("aligned", aligned_weight(), aligned_input(), aligned_upstream()),
                           ("edge", edge_weight(), edge_input(), edge_upstream())):
        out[f"{name}_weight"] = W
        out[f"{name}_input"] = X
        out[f"{name}_upstream"] = dY
        for enc, w in (("fp32", ref.quantize_nf4(W, 32)),
                       ("dq", ref.quantize_nf4_double_quantized(W, 32, 32))):
            p = f"{name}_{enc}"
            out.update(payload_arrays(p, w))
            out[f"{p}_dequant"] = ref.dequantize(w)
            out[f"{p}_forward"] = ref.linear_forward(w, X)
            out[f"{p}_backward"] = ref.linear_input_backward(w, dY)

    # -- paged decode fixture of the reference nn-backend test ---------------------
    qv, kv, vv, query, key_pages, value_pages, table, time = paged_fixture()
    _, causal_ctx = ref.materialized_causal_forward(qv, kv, vv)
    out["paged_query"] = query
    out["paged_key_pages"] = key_pages
    out["paged_value_pages"] = value_pages
    out["paged_table"] = table
    out["paged_seq_len"] = np.array([time], np.int64)
    out["paged_expected_causal_last_row"] = causal_ctx[0, :, time - 1, :]
    out["paged_reference_context"] = ref.paged_decode(query, key_pages, value_pages, table, time)

    # -- seeded random cases, reference outputs ------------------------------------
    c = seeded_cases()
    # Config 1 of the baseline: X[64,512] ~ N(0,1), W[1024,512] ~ N(0,0.02^2), block 64, FP32 scales.
    w1 = ref.quantize_nf4(c["W1"], 64)
    out["c1_codes_xor"] = np.array([int(np.bitwise_xor.reduce(w1.codes.view(np.uint32)))], np.uint64)
    out["c1_scales"] = w1.fp32_scales
    out["c1_forward_rows0_8"] = ref.linear_forward(w1, c["X1"])[:8]
    w1d = ref.quantize_nf4_double_quantized(c["W1"], 64, 256)
    out["c1_dq_scale_codes"] = w1d.scale_codes
    out["c1_dq_second_level"] = w1d.second_level
    out["c1_dq_offset"] = np.array([w1d.offset], np.float32)
    out["c1_dq_forward_rows0_8"] = ref.linear_forward(w1d, c["X1"])[:8]
    out["c1_dq_backward"] = ref.linear_input_backward(w1d, c["dY1"])
    # One GQA-shaped sequence (32 query / 8 KV heads) through the unmodified operator.
    out["gqa_context"] = ref.paged_decode_gqa(c["q"], c["K"], c["V"], c["table"][None, :],
                                              np.array([c["seq_len"]], np.uint32))

    # -- decode-step primitives around the hot path (reference entry points in oracle/ref_bridge.cpp)
    g = decode_glue_inputs()
    out["glue_rms"] = ref.rms_norm(g["rms_x"], g["rms_scale"], 1e-5)
    for pos in ROPE_POSITIONS:
        out[f"glue_rope_{pos}"] = ref.rope(g["rope_x"], pos, 1e4)
    out["glue_silu"] = ref.silu_mul(g["silu_gate"])
    out["glue_swiglu_hidden"] = ref.silu_mul(g["silu_gate"], g["silu_up"])
    out["glue_greedy"] = np.array([ref.greedy(row) for row in g["greedy_logits"]], np.int64)
    # one sequence fed token by token through the reference's paged KV cache (page 4, 5 pages): k is
    # rotated by the reference first, so this pins RoPE + page append + paged attention end to end
    steps = g["cache_q"].shape[0]
    k_rot = np.stack([ref.rope(g["cache_k"][t][None, :, None, :], t, 1e4)[0, :, 0, :] for t in range(steps)])
    q_rot = np.stack([ref.rope(g["cache_q"][t][None, :, None, :], t, 1e4)[0, :, 0, :] for t in range(steps)])
    out["glue_cache_context"] = ref.paged_cache_decode(q_rot, k_rot, g["cache_v"], 4, 5)

    # -- LoRA branch of a Linear and the adapted NF4 linear (base + branch) ---------------------
    lo = lora_inputs()
    out["lora_branch"] = ref.lora_forward(lo["x"], lo["a"], lo["b"], float(lo["scale"]))
    wl = ref.quantize_nf4(lo["w"], 32)
    out["lora_adapted_linear"] = ref.linear_forward(wl, lo["x"]) + out["lora_branch"]

    # -- canonical packed model state written by the reference (RTNF4S1) ---------------------
    for name, scale_block in (("rtnf4_dq", 32), ("rtnf4_f32", 0)):
        stream, dump = ref.packed_model_fixture(32, 16, 64, 2, 2, 128, 64, scale_block, 7)
        out[f"{name}_stream"] = stream
        out[f"{name}_fields"] = dump

    np.savez_compressed(OUT / "reference_vectors.npz", **out)
    size = (OUT / "reference_vectors.npz").stat().st_size
    print(f"wrote {len(out)} arrays, {size} bytes")


if __name__ == "__main__":
    main()
