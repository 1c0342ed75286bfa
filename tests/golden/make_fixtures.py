"""Writes the golden fixtures of this directory.  Run from the repository root:

    python tests/golden/make_fixtures.py

Nothing here imports the library or the oracle: the fixtures are built from the reference's published
formats and known answers alone, so that both implementations can be checked against them.

* ``snapshot_v1_tiny.bin.gz`` -- an 'MFLX' version-1 snapshot laid out by hand from the wire format of
  crates/moeflux/src/riir/state_snapshot.rs:1-31 (C twin: metal_infer/infer.m:8671-8692): little-endian header
  of eight u32 {magic 0x4D464C58, version, num_layers, full_attn_interval, num_kv_heads, head_dim,
  linear_conv_bytes, linear_ssm_bytes}, then per layer either conv_state f32 [3][conv_dim] + ssm_state f32
  [v_heads][128][128] (GatedDeltaNet layer) or i32 len + K f32 [len][kv_dim] + V f32 [len][kv_dim]
  (full-attention layer: every full_attn_interval-th).  Geometry: 4 layers, interval 4, 2 kv heads of 256 dims,
  2 k-heads and 4 v-heads of 128 dims (conv_dim 1024), kv length 3.  All payload is zero except the probe
  values listed in ``fixtures.json`` (first and last element of every block), which pin the offsets.
* ``fixtures.json`` -- the probes above, and the known answers of the reference's unit tests of
  ``dequant_matvec_4bit_cpu`` (crates/moeflux/src/riir/cpu_matvec.rs:366-451), transcribed from that file.
"""
import gzip
import json
import os
import struct

HERE = os.path.dirname(os.path.abspath(__file__))

NUM_LAYERS, INTERVAL, KV_HEADS, HEAD_DIM = 4, 4, 2, 256
K_HEADS, V_HEADS, LIN_DIM, CONV_TAPS = 2, 4, 128, 4
CONV_DIM = 2 * K_HEADS * LIN_DIM + V_HEADS * LIN_DIM
KV_DIM = KV_HEADS * HEAD_DIM
SSM_ELEMS = V_HEADS * LIN_DIM * LIN_DIM
KV_LEN = 3


def build_snapshot():
    conv_bytes, ssm_bytes = (CONV_TAPS - 1) * CONV_DIM * 4, SSM_ELEMS * 4
    buf = bytearray(struct.pack("<8I", 0x4D464C58, 1, NUM_LAYERS, INTERVAL, KV_HEADS, HEAD_DIM, conv_bytes, ssm_bytes))
    probes = []

    def block(name, layer, n_floats):
        start = len(buf)
        buf.extend(bytes(4 * n_floats))
        for idx, val in ((0, 1.0 + layer + 0.25 * len(probes)), (n_floats - 1, -(2.0 + layer) - 0.5 * len(probes))):
            struct.pack_into("<f", buf, start + 4 * idx, val)
            probes.append({"layer": layer, "block": name, "index": idx, "value": struct.unpack("<f", struct.pack("<f", val))[0],
                           "byte_offset": start + 4 * idx})

    for layer in range(NUM_LAYERS):
        if (layer + 1) % INTERVAL == 0:
            buf.extend(struct.pack("<i", KV_LEN))
            block("k", layer, KV_LEN * KV_DIM)
            block("v", layer, KV_LEN * KV_DIM)
        else:
            block("conv", layer, (CONV_TAPS - 1) * CONV_DIM)
            block("ssm", layer, SSM_ELEMS)
    return bytes(buf), probes


def main():
    data, probes = build_snapshot()
    with gzip.GzipFile(os.path.join(HERE, "snapshot_v1_tiny.bin.gz"), "wb", mtime=0) as f:
        f.write(data)
    fixtures = {
        "snapshot_v1_tiny": {
            "geometry": {"num_layers": NUM_LAYERS, "full_attn_interval": INTERVAL, "num_kv_heads": KV_HEADS,
                         "head_dim": HEAD_DIM, "linear_num_k_heads": K_HEADS, "linear_num_v_heads": V_HEADS},
            "kv_len": KV_LEN, "size": len(data), "probes": probes},
        # crates/moeflux/src/riir/cpu_matvec.rs:366-451; scales and biases are bf16 bit patterns
        "dequant_matvec_4bit": [
            {"name": "dequant_matvec_all_ones", "in_dim": 64, "out_dim": 1, "packed_word": 0x11111111, "scale": 0x3F80,
             "bias": 0x0000, "x": 1.0, "expected": [64.0]},
            {"name": "zero_input_yields_zero_output", "in_dim": 64, "out_dim": 2, "packed_word": 0xFFFFFFFF, "scale": 0x3F80,
             "bias": 0x3F80, "x": 0.0, "expected": [0.0, 0.0]},
            {"name": "bias_only_path", "in_dim": 64, "out_dim": 1, "packed_word": 0x00000000, "scale": 0x40A0,
             "bias": 0x4000, "x": 1.0, "expected": [128.0]},
        ],
    }
    with open(os.path.join(HERE, "fixtures.json"), "w") as f:
        json.dump(fixtures, f, indent=1)
        f.write("\n")
    print("wrote", len(data), "snapshot bytes,", len(probes), "probes")


if __name__ == "__main__":
    main()
