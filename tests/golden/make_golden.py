"""Regenerates the fixtures in this directory.  Run in a container that has the
reference checkout (it is imported by file path; nothing from it is copied):

    python tests/golden/make_golden.py /path/to/reference

ref_codec.npz   outputs of the REFERENCE's own Python for inputs chosen here:
                 - f32_vec_to_bf16_u16 (moe_infer/helpers/quantize_from_hf.py:46-53),
                   the same expression as src/dtype.rs:85-89
                 - dequant_int4        (moe_infer/dequantize.py:42-63)
                 - _expert_layout      (moe_infer/dequantize.py:142-160)
                 - _dequant_expert_section (moe_infer/dequantize.py:163-175) applied
                   to a blob assembled by the CPU oracle -> pins section order/offsets
packer_kat.npz  known-answer vectors of the packer produced by the CPU oracle
                (the reference ships none; these pin the restatement of
                src/dtype.rs:102-135 against regressions and are what the GPU packer
                is compared with byte for byte).
"""
import importlib.util
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
import oracle  # noqa: E402


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def packer_cases():
    """Edge cases of quant_f32_to_int4, one or more 64-wide groups each."""
    rng = np.random.Generator(np.random.PCG64(20240601))
    cases = {}
    cases["constant_group"] = np.full((1, 64), 0.125, np.float32)
    cases["constant_zero_free"] = np.full((1, 64), -3.5, np.float32)
    ramp = (np.arange(64, dtype=np.float32) / 63.0).reshape(1, 64)
    cases["ramp_0_1"] = ramp
    # values exactly half-way between two levels: min 0, max 15 -> scale 1, v = k + 0.5
    half = np.zeros((1, 64), np.float32)
    half[0, :16] = np.arange(16, dtype=np.float32)
    half[0, 16:31] = np.arange(15, dtype=np.float32) + 0.5
    half[0, 63] = 15.0
    cases["half_way_levels"] = half
    cases["negative_only"] = -np.abs(rng.standard_normal((2, 128)).astype(np.float32)) - 0.01
    cases["positive_only"] = np.abs(rng.standard_normal((2, 128)).astype(np.float32)) + 0.01
    cases["mixed_sign"] = (rng.standard_normal((4, 256)) * 0.02).astype(np.float32)
    out = (rng.standard_normal((4, 256)) * 0.02).astype(np.float32)
    out[0, 5] = 0.4
    out[1, 70] = -0.4
    out[2, 128] = 0.4
    out[2, 129] = -0.4
    cases["outliers_20_sigma"] = out
    # scales/biases whose f32 bits exercise the bf16 rounding rule: craft min/max pairs
    quirk = np.zeros((8, 64), np.float32)
    pats = [0x3F808002, 0x3F808001, 0x3F818000, 0x3F80C000, 0x3F7F8001, 0x3F7FFFFF, 0xBF808002, 0x3E008000]
    for r, pat in enumerate(pats):
        vmin = np.array([pat], np.uint32).view(np.float32)[0]
        quirk[r, :] = vmin
        quirk[r, 1::2] = vmin + np.float32(abs(vmin)) * np.float32(0.37) + np.float32(1e-3)
    cases["bf16_rounding_of_scale_bias"] = quirk
    tiny = (rng.standard_normal((2, 64)) * 1e-30).astype(np.float32)
    cases["tiny_magnitudes"] = tiny
    big = (rng.standard_normal((2, 64)) * 1e30).astype(np.float32)
    cases["huge_magnitudes"] = big
    cases["random_n02"] = (rng.standard_normal((16, 512)) * 0.02).astype(np.float32)
    sin = np.sin(np.arange(2 * 128, dtype=np.float32)).reshape(2, 128)  # the reference's own round-trip input
    cases["reference_roundtrip_input_sin"] = sin
    return cases


def main():
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <path to a checkout of the reference project>")
    ref = sys.argv[1]
    deq = _load(os.path.join(ref, "moe_infer", "dequantize.py"), "ref_dequantize")
    qhf = _load(os.path.join(ref, "moe_infer", "helpers", "quantize_from_hf.py"), "ref_quantize_from_hf")
    rng = np.random.Generator(np.random.PCG64(7))

    # bf16 rounding: hand-picked bit patterns + random
    special = np.array([0x3F808002, 0x3F808000, 0x3F808001, 0x3F818000, 0x3F818001, 0x3F80FFFF, 0x3F7FFFFF,
                        0x3F7F8000, 0x3F7F8001, 0x00000000, 0x80000000, 0x00008001, 0x7F7FFFFF, 0x7F7F8001,
                        0xBF808002, 0xBF818000, 0x3DCCCCCD, 0x3E4CCCCD], np.uint32)
    rnd = rng.integers(0, 2**32, size=4096, dtype=np.uint64).astype(np.uint32)
    exp = (rnd >> 23) & 0xFF
    rnd = rnd[exp != 0xFF]  # drop Inf/NaN
    bf_in = np.concatenate([special, rnd]).astype(np.uint32)
    bf_out = qhf.f32_vec_to_bf16_u16(bf_in.view(np.float32).copy())

    # dequantiser
    dq_w = rng.integers(0, 2**32, size=(4, 16), dtype=np.uint64).astype(np.uint32)
    dq_s = oracle.f32_to_bf16(np.abs(rng.standard_normal((4, 2)).astype(np.float32)) * 0.01)
    dq_b = oracle.f32_to_bf16(rng.standard_normal((4, 2)).astype(np.float32) * 0.05)
    dq_out = deq.dequant_int4(dq_w.ravel(), dq_s.ravel(), dq_b.ravel(), 4, 128).astype(np.float32)

    # layout
    layouts_in = np.array([[2048, 512, 64], [1024, 256, 64], [128, 64, 64]], np.int64)
    keys = ["gate_w_off", "gate_s_off", "gate_b_off", "up_w_off", "up_s_off", "up_b_off",
            "down_w_off", "down_s_off", "down_b_off", "expert_size"]
    layouts_out = np.array([[deq._expert_layout(int(h), int(m), int(g))[k] for k in keys]
                            for h, m, g in layouts_in], np.int64)

    # blob section order: oracle-assembled blob decoded by the reference
    hd, mi, E = 128, 64, 3
    gu = (rng.standard_normal((E, 2 * mi, hd)) * 0.02).astype(np.float32)
    dn = (rng.standard_normal((E, hd, mi)) * 0.02).astype(np.float32)
    blob = oracle.pack_experts_layer(gu, dn)
    lay = deq._expert_layout(hd, mi, 64)
    sec = []
    for e in range(E):
        mv = memoryview(blob.tobytes())[e * lay["expert_size"]:(e + 1) * lay["expert_size"]]
        sec.append([deq._dequant_expert_section(mv, lay["gate_w_off"], mi, hd),
                    deq._dequant_expert_section(mv, lay["up_w_off"], mi, hd)])
    sec_gate = np.stack([s[0] for s in sec]).astype(np.float32)
    sec_up = np.stack([s[1] for s in sec]).astype(np.float32)
    sec_down = np.stack([deq._dequant_expert_section(
        memoryview(blob.tobytes())[e * lay["expert_size"]:(e + 1) * lay["expert_size"]], lay["down_w_off"], hd, mi)
        for e in range(E)]).astype(np.float32)

    np.savez_compressed(os.path.join(HERE, "ref_codec.npz"), bf16_in=bf_in, bf16_out=bf_out.astype(np.uint16),
                        dq_w=dq_w, dq_s=dq_s, dq_b=dq_b, dq_out=dq_out, layouts_in=layouts_in,
                        layouts_out=layouts_out, blob_gate_up=gu, blob_down=dn, blob_bytes=blob,
                        blob_sec_gate=sec_gate, blob_sec_up=sec_up, blob_sec_down=sec_down)

    kat = {}
    for name, v in packer_cases().items():
        w, s, b = oracle.quant_int4(v)
        kat[name + ".in"] = v
        kat[name + ".w"] = w
        kat[name + ".s"] = s
        kat[name + ".b"] = b
    np.savez_compressed(os.path.join(HERE, "packer_kat.npz"), **kat)
    print("wrote", os.listdir(HERE))


if __name__ == "__main__":
    main()
