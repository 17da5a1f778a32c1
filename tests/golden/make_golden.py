#!/usr/bin/env python3
"""Makes tests/golden/reference_primitives.json: the outputs of hardenedlinux/SonicBoom's own
CPU primitives on small seeded inputs, for tests/test_golden.py to hold the plain
implementation against.

The reference's model code (core/src/model/emit.cpp and the planner behind it) cannot be built
without its MLIR submodule and GGUF models, but its float32 CPU primitives compile on their own.
This script compiles them IN PLACE from a checkout of the reference (nothing of it is copied
into this repository), together with a small driver that calls them in the order the emitter
uses for one Qwen2 block (core/src/model/emit.cpp:255-308, 364-374, 436-459, 512-523):

    rms_norm, matvec_f32 + add_bias (q, k, v), rope_neox_heads (q, k),
    scaled_dot_product_attention (causal, grouped heads; also with a window) and decode_attention,
    matvec_f32 (o), add, rms_norm, matvec_f32 (up, gate), silu, mul, matvec_f32 (down), add,
    final rms_norm and head matvec; then argmax, philox4x32_10 and sample_token.

Unlike the reference's graph, the driver does not round K and V through float16 (the reference's
CastFp16 nodes, emit.cpp:291-293): the golden values pin the formulas, not that storage choice.

    python tests/golden/make_golden.py <checkout of hardenedlinux/SonicBoom>

Needs g++ with C++23.  The JSON it writes is committed; the test does not need the reference.
"""
import json
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent

# a tiny one-layer model: 3 query heads over 1 key/value head of 8, width 24, intermediate 40
CFG = dict(d=24, hq=3, hkv=1, hd=8, ff=40, vocab=50, n=7, eps=1e-5, theta=10000.0, window=3)

DRIVER = r'''
#include <sonicboom/nn/norm.h>
#include <sonicboom/nn/rope.h>
#include <sonicboom/nn/attention.h>
#include <sonicboom/nn/activation.h>
#include <sonicboom/nn/elementwise.h>
#include <sonicboom/nn/matmul.h>
#include <sonicboom/nn/sampling.h>
#include <sonicboom/compiler/ReduceMode.h>
#include <cmath>
#include <cstdio>
#include <cstdint>
#include <optional>
#include <string>
#include <vector>
namespace sonicboom::planner {            // the one symbol the primitives need from the planner
compiler::ReduceMode cpu_reduce_mode() { return compiler::ReduceMode::F64; }
}
using namespace sonicboom;
using V = std::vector<float>;
static V rd(FILE* f, size_t n) { V v(n); if (fread(v.data(), 4, n, f) != n) { perror("read"); exit(1); } return v; }
static void out(const char* name, const V& v, bool last = false) {
  printf("\"%s\": [", name);
  for (size_t i = 0; i < v.size(); ++i) printf("%s%.9g", i ? "," : "", v[i]);
  printf("]%s\n", last ? "" : ",");
}
int main(int argc, char** argv) {
  FILE* f = fopen(argv[1], "rb");
  int32_t h[8]; if (fread(h, 4, 8, f) != 8) return 1;
  const uint64_t d = h[0], hq = h[1], hkv = h[2], hd = h[3], ff = h[4], vocab = h[5], n = h[6], window = h[7];
  float fl[2]; if (fread(fl, 4, 2, f) != 2) return 1;
  const float eps = fl[0], theta = fl[1];
  const uint64_t qw = hq * hd, kvw = hkv * hd;
  V x = rd(f, n * d), wn1 = rd(f, d), wq = rd(f, qw * d), bq = rd(f, qw), wk = rd(f, kvw * d), bk = rd(f, kvw),
    wv = rd(f, kvw * d), bv = rd(f, kvw), wo = rd(f, d * qw), wn2 = rd(f, d), wup = rd(f, ff * d),
    wgate = rd(f, ff * d), wdown = rd(f, d * ff), wnf = rd(f, d), whead = rd(f, vocab * d);
  V hn(n * d), q(n * qw), k(n * kvw), v(n * kvw);
  for (uint64_t t = 0; t < n; ++t) {
    std::span<float> hr(hn.data() + t * d, d);
    nn::rms_norm({x.data() + t * d, d}, wn1, eps, hr);
    std::span<float> qr(q.data() + t * qw, qw), kr(k.data() + t * kvw, kvw), vr(v.data() + t * kvw, kvw);
    nn::matvec_f32(wq, d, hr, qr); nn::add_bias(qr, bq, qr);
    nn::rope_neox_heads(qr, hd, t, theta, 1.0f, {}, 0);
    nn::matvec_f32(wk, d, hr, kr); nn::matvec_f32(wv, d, hr, vr);
    nn::add_bias(kr, bk, kr); nn::add_bias(vr, bv, vr);
    nn::rope_neox_heads(kr, hd, t, theta, 1.0f, {}, 0);
  }
  const float scale = 1.0f / std::sqrt(float(hd));
  V att(n * qw), attw(n * qw), dec(qw);
  nn::scaled_dot_product_attention(q, n, k, v, n, hq, hkv, hd, true, 0, 0.0f, scale, att);
  nn::scaled_dot_product_attention(q, n, k, v, n, hq, hkv, hd, true, window, 0.0f, scale, attw);
  nn::decode_attention({q.data() + (n - 1) * qw, qw}, k, v, n - 1, n, hq, hkv, hd, 0, scale, dec);
  V x2(n * d), logits(n * vocab), f1(n * d), act(n * ff);
  for (uint64_t t = 0; t < n; ++t) {
    V o(d), up(ff), gate(ff), dn(d), hf(d);
    nn::matvec_f32(wo, qw, {att.data() + t * qw, qw}, o);
    for (uint64_t i = 0; i < d; ++i) o[i] += x[t * d + i];                      // x1 = o + residual
    nn::rms_norm(o, wn2, eps, {f1.data() + t * d, d});
    nn::matvec_f32(wup, d, {f1.data() + t * d, d}, up);
    nn::matvec_f32(wgate, d, {f1.data() + t * d, d}, gate);
    nn::silu(gate, gate);
    for (uint64_t i = 0; i < ff; ++i) act[t * ff + i] = gate[i] * up[i];
    nn::matvec_f32(wdown, ff, {act.data() + t * ff, ff}, dn);
    for (uint64_t i = 0; i < d; ++i) x2[t * d + i] = dn[i] + o[i];             // x2 = ffn + x1
    nn::rms_norm({x2.data() + t * d, d}, wnf, eps, hf);
    nn::matvec_f32(whead, d, hf, {logits.data() + t * vocab, vocab});
  }
  printf("{\n");
  out("normed", hn); out("q_rotated", q); out("k_rotated", k); out("v", v);
  out("attention", att); out("attention_window", attw); out("decode_attention", dec);
  out("swiglu_act", act); out("block_out", x2); out("logits", logits);
  // sampling on the last row's logits
  std::span<const float> last(logits.data() + (n - 1) * vocab, vocab);
  std::vector<int64_t> history = {3, 7, 7, 11, 3, 7};
  V picks;
  picks.push_back(float(nn::argmax(last)));
  struct Case { float t; uint32_t k; float p, minp; uint64_t seed; float rp, pp, fp; uint32_t last_n; };
  const Case cases[] = {{0.0f, 0, 1.0f, 0.0f, 0, 1.0f, 0, 0, 64}, {0.8f, 0, 1.0f, 0.0f, 5, 1.0f, 0, 0, 64},
                        {1.5f, 5, 1.0f, 0.0f, 1, 1.0f, 0, 0, 64}, {1.0f, 0, 0.6f, 0.0f, 9, 1.0f, 0, 0, 64},
                        {0.7f, 0, 1.0f, 0.2f, 3, 1.0f, 0, 0, 64}, {0.9f, 0, 1.0f, 0.0f, 4, 1.3f, 0.5f, 0.25f, 4},
                        {0.0f, 0, 1.0f, 0.0f, 0, 5.0f, 9.0f, 0, 64}, {2.0f, 20, 0.9f, 0.01f, 1ull << 40, 1.1f, 0.1f, 0.1f, 3}};
  for (const Case& c : cases)
    for (uint64_t pos : {uint64_t(0), uint64_t(17), (uint64_t(1) << 33) + 1}) {
      nn::SamplingParams sp; sp.temperature = c.t; sp.top_k = c.k; sp.top_p = c.p; sp.min_p = c.minp;
      sp.seed = c.seed; sp.repeat_penalty = c.rp; sp.presence_penalty = c.pp; sp.frequency_penalty = c.fp;
      sp.repeat_last_n = c.last_n;
      picks.push_back(float(nn::sample_token(last, sp, pos, history, {})));
    }
  out("sample_tokens", picks);
  auto ph = nn::philox4x32_10({1, 2, 3, 4}, 0x123456789abcdefull);
  out("philox", {float(ph[0] >> 16), float(ph[0] & 0xffff), float(ph[1] >> 16), float(ph[1] & 0xffff)}, true);
  printf("}\n");
  return 0;
}
'''


SEED = 20240607


def make_inputs():
    """The seeded inputs, in the order the driver reads them: {name: float32 array}."""
    c = CFG
    rng = np.random.default_rng(SEED)
    qw, kvw = c["hq"] * c["hd"], c["hkv"] * c["hd"]
    shapes = [("x", (c["n"], c["d"]), 1.0), ("wn1", (c["d"],), None), ("wq", (qw, c["d"]), 0.3), ("bq", (qw,), 0.2),
              ("wk", (kvw, c["d"]), 0.3), ("bk", (kvw,), 0.2), ("wv", (kvw, c["d"]), 0.3), ("bv", (kvw,), 0.2),
              ("wo", (c["d"], qw), 0.3), ("wn2", (c["d"],), None), ("wup", (c["ff"], c["d"]), 0.3),
              ("wgate", (c["ff"], c["d"]), 0.3), ("wdown", (c["d"], c["ff"]), 0.3), ("wnf", (c["d"],), None),
              ("whead", (c["vocab"], c["d"]), 0.5)]
    tensors = {}
    for name, shape, std in shapes:
        t = rng.standard_normal(shape).astype(np.float32)
        tensors[name] = (1.0 + 0.1 * t).astype(np.float32) if std is None else (std * t).astype(np.float32)
    return tensors


def main() -> int:
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    REF = Path(sys.argv[1])
    c = CFG
    tensors = make_inputs()
    with tempfile.TemporaryDirectory() as tmp:
        tmp = Path(tmp)
        with open(tmp / "in.bin", "wb") as f:
            f.write(np.asarray([c["d"], c["hq"], c["hkv"], c["hd"], c["ff"], c["vocab"], c["n"], c["window"]],
                               dtype=np.int32).tobytes())
            f.write(np.asarray([c["eps"], c["theta"]], dtype=np.float32).tobytes())
            for name in tensors:
                f.write(tensors[name].tobytes())
        (tmp / "driver.cpp").write_text(DRIVER)
        srcs = [REF / "core/src/nn" / s for s in
                ("norm.cpp", "rope.cpp", "attention.cpp", "activation.cpp", "elementwise.cpp", "matmul.cpp",
                 "sampling.cpp")] + [REF / "core/src/thread_pool.cpp"]
        cmd = ["g++", "-std=c++23", "-O1", "-I", str(REF / "core/include"), "-I", str(REF / "core/compiler/include"),
               "-I", str(REF / "core/src"), str(tmp / "driver.cpp"), *map(str, srcs), "-lpthread", "-o",
               str(tmp / "driver")]
        subprocess.run(cmd, check=True)
        out = subprocess.run([str(tmp / "driver"), str(tmp / "in.bin")], check=True, capture_output=True,
                             text=True).stdout
    golden = json.loads(out)
    golden["config"] = c
    golden["seed"] = SEED                    # the inputs are remade from it by make_inputs()
    golden["made_by"] = "tests/golden/make_golden.py from hardenedlinux/SonicBoom core/src/nn/*.cpp (v0.0.6)"
    (HERE / "reference_primitives.json").write_text(json.dumps(golden))
    print(f"wrote {HERE / 'reference_primitives.json'} ({len(json.dumps(golden))} bytes)")
    return 0


if __name__ == "__main__":
    sys.exit(main())
