#!/usr/bin/env python3
"""Anchors tests/plain_qwen3.py against the reference's own compiled CPU code, once.

Builds laik/vllm-cpp's src/model.cpp (with quantization.cpp and quant_loader.cpp) and a
twenty-line driver around its load_model_safetensors + forward_cpu, writes a tiny random model
in a temporary folder, runs the reference on several prefixes of one token list and stores the
last-position logits in tests/golden/reference_logits.json together with everything needed to
rebuild the same model (seed and sizes).  tests/test_plain.py rebuilds the model and compares.

The reference's CPU forward is not the intended Qwen3 (see the switches of plain_qwen3.forward),
so the model is made such that its accidents do not show or can be switched on in the plain
implementation:
  * it never applies q_norm / k_norm                       -> plain runs with qk_norm=False
  * it rotates interleaved lane pairs (src/model.cpp:983)  -> plain runs with rope_interleaved_lanes=True
  * it ignores rope_theta and uses 1e6 (src/config.h:43)   -> config says rope_theta 1e6
  * its number reader has no exponent (src/model.cpp:340)  -> rms_norm_eps is spelled 0.000001
  * it finds the final norm by substring and lands on layer 0's input norm (src/model.cpp:392-400)
                                                           -> model.norm.weight is a copy of that tensor
  * it sizes the Q projection by hidden_size (:1206)        -> heads * head_dim == hidden_size
  * its down projection runs in place (:1243)               -> plain runs with down_in_place=True

Usage: python tests/golden/make_golden.py /path/to/laik-vllm-cpp
"""
import json
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))

SPEC = dict(seed=7, vocab_size=160, hidden_size=64, intermediate_size=112, num_hidden_layers=2,
            num_attention_heads=4, num_key_value_heads=2, head_dim=16, tokens_seed=8, n_tokens=12,
            prefixes=[1, 2, 5, 12])

DRIVER = r'''
#include "model.h"
#include <iostream>
#include <iomanip>
#include <sstream>
int main(int argc, char** argv) {
    Qwen36Model model = load_model_safetensors(argv[1]);
    std::vector<int32_t> ids;
    { std::istringstream iss(argv[2]); std::string t; while (std::getline(iss, t, ',')) ids.push_back(std::stoi(t)); }
    std::cout << std::setprecision(9);
    for (int a = 3; a < argc; ++a) {
        int n = std::stoi(argv[a]);
        std::vector<int32_t> prefix(ids.begin(), ids.begin() + n);
        auto logits = forward_cpu(model, prefix, 1, false);
        std::cout << "LOGITS " << n;
        for (size_t i = 0; i < logits.size(); ++i) std::cout << " " << logits[i];
        std::cout << std::endl;
    }
    return 0;
}
'''


def make_weights(spec):
    """The tiny model's tensors (float32), a pure function of the spec."""
    rng = np.random.default_rng(spec["seed"])
    H, I, V = spec["hidden_size"], spec["intermediate_size"], spec["vocab_size"]
    nh, nkv, hd = spec["num_attention_heads"], spec["num_key_value_heads"], spec["head_dim"]
    w = {}

    def mat(name, shape):
        w[name] = rng.normal(0, 0.05, size=shape).astype(np.float32)

    def gain(name, n):
        w[name] = (1 + rng.normal(0, 0.1, size=n)).astype(np.float32)

    mat("model.embed_tokens.weight", (V, H))
    for l in range(spec["num_hidden_layers"]):
        p = f"model.layers.{l}."
        gain(p + "input_layernorm.weight", H)
        mat(p + "self_attn.q_proj.weight", (nh * hd, H))
        mat(p + "self_attn.k_proj.weight", (nkv * hd, H))
        mat(p + "self_attn.v_proj.weight", (nkv * hd, H))
        mat(p + "self_attn.o_proj.weight", (H, nh * hd))
        gain(p + "self_attn.q_norm.weight", hd)
        gain(p + "self_attn.k_norm.weight", hd)
        gain(p + "post_attention_layernorm.weight", H)
        mat(p + "mlp.gate_proj.weight", (I, H))
        mat(p + "mlp.up_proj.weight", (I, H))
        mat(p + "mlp.down_proj.weight", (H, I))
    w["model.norm.weight"] = w["model.layers.0.input_layernorm.weight"].copy()
    mat("lm_head.weight", (V, H))
    return w


def make_config(spec):
    return {"architectures": ["Qwen3ForCausalLM"], "vocab_size": spec["vocab_size"], "hidden_size": spec["hidden_size"],
            "intermediate_size": spec["intermediate_size"], "num_hidden_layers": spec["num_hidden_layers"],
            "num_attention_heads": spec["num_attention_heads"], "num_key_value_heads": spec["num_key_value_heads"],
            "head_dim": spec["head_dim"], "max_position_embeddings": 64, "rope_theta": 1000000.0,
            "rms_norm_eps": 1e-6, "tie_word_embeddings": False}


def make_tokens(spec):
    return np.random.default_rng(spec["tokens_seed"]).integers(0, spec["vocab_size"], spec["n_tokens"]).tolist()


def write_model(folder, spec):
    import struct
    w = make_weights(spec)
    cfg = make_config(spec)
    text = json.dumps(cfg, indent=1).replace("1e-06", "0.000001")   # the reference's reader has no exponent
    (folder / "config.json").write_text(text)
    header, off = {}, 0
    for name in sorted(w):
        n = w[name].nbytes
        header[name] = {"dtype": "F32", "shape": list(w[name].shape), "data_offsets": [off, off + n]}
        off += n
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(folder / "model.safetensors", "wb") as f:
        f.write(struct.pack("<Q", len(blob)) + blob)
        for name in sorted(w):
            f.write(w[name].tobytes())


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py <folder of a laik/vllm-cpp checkout>")
    ref = Path(sys.argv[1])
    src = ref / "src"
    with tempfile.TemporaryDirectory() as tmp:
        tmp = Path(tmp)
        (tmp / "driver.cpp").write_text(DRIVER)
        subprocess.run(["g++", "-std=c++20", "-O2", f"-I{src}", str(tmp / "driver.cpp"), str(src / "model.cpp"),
                        str(src / "quantization.cpp"), str(src / "quant_loader.cpp"), "-o", str(tmp / "refdrv")], check=True)
        model = tmp / "model"
        model.mkdir()
        write_model(model, SPEC)
        toks = make_tokens(SPEC)
        out = subprocess.run([str(tmp / "refdrv"), str(model), ",".join(map(str, toks)), *map(str, SPEC["prefixes"])],
                             check=True, capture_output=True, text=True).stdout
    logits = {}
    for line in out.splitlines():
        if line.startswith("LOGITS "):
            parts = line.split()
            logits[parts[1]] = [float(x) for x in parts[2:]]
    assert sorted(map(int, logits)) == sorted(SPEC["prefixes"]), out[-2000:]
    (HERE / "reference_logits.json").write_text(json.dumps({"spec": SPEC, "tokens": toks, "logits": logits}))
    print("wrote", HERE / "reference_logits.json", {k: len(v) for k, v in logits.items()})


if __name__ == "__main__":
    main()
