#!/usr/bin/env python3
"""Makes tests/golden/*.npz: logits of the reference's own model code on tiny random models.

What it does, on the CPU, touching nothing outside a temporary folder:

1. copies the reference source tree and applies two portability shims (the non-Windows branch of
   src/core/thread_pool.cpp lacks two helpers its constructor calls; src/memory/system_ram.cpp
   has no non-Windows memory query, so the loader's budget is zero) - no arithmetic is touched;
2. builds it with cmake (Vulkan off) and compiles tests/golden/reference_driver.cpp against
   libtge_core.a;
3. writes the tiny configurations A and B of tests/conftest.py as model folders with this
   package's random-weights mode, and converts each to a float32 GGUF file with the reference's
   tensor names (src/models/qwen2.cpp:411-523) and metadata keys (src/models/qwen2.cpp:222-250);
4. runs the reference (scalar attention, scalar kernels, one thread): a whole prompt, decode
   steps after it, an all-rows batch, and a mixed batch of two sequences;
5. stores tokens, the script, the logits and a hash of the weights in tests/golden/tiny_<name>.npz.

6. runs the reference's sampler (src/models/sampling.cpp: sample_token; tests/golden/reference_sampler_driver.cpp)
   on seeded logits rows with every option it has, a few hundred draws, and stores the picks in
   tests/golden/sampler.npz.

tests/test_plain_vs_golden.py then checks the plain implementation against these files.

    python tests/golden/make_golden.py --reference PATH_TO_THE_REFERENCE_CHECKOUT
"""
import argparse
import hashlib
import os
import random
import shutil
import struct
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def shim(tree):
    path = os.path.join(tree, "src/core/thread_pool.cpp")
    text = open(path).read()
    old = "#else\ninline void pin_worker_to_p_core(int /*worker_index*/) {}\n#endif"
    assert old in text, "thread_pool.cpp changed: review the shim"
    text = text.replace(old, "#else\ninline std::vector<int> p_core_logicals() { return {}; }\n"
                             "inline void pin_worker_to_p_core(const std::vector<int>&, int) {}\n#endif")
    open(path, "w").write(text)
    path = os.path.join(tree, "src/memory/system_ram.cpp")
    text = open(path).read()
    old = "  memory.allocation_granularity = info.dwAllocationGranularity;\n#endif\n"
    assert old in text, "system_ram.cpp changed: review the shim"
    text = text.replace(old, "  memory.allocation_granularity = info.dwAllocationGranularity;\n#else\n  {\n"
                             "    const long page = sysconf(_SC_PAGESIZE);\n"
                             "    memory.total_physical = static_cast<std::uint64_t>(sysconf(_SC_PHYS_PAGES)) * page;\n"
                             "    memory.available_physical = static_cast<std::uint64_t>(sysconf(_SC_AVPHYS_PAGES)) * page;\n"
                             "    memory.total_commit = memory.total_physical;\n"
                             "    memory.available_commit = memory.available_physical;\n"
                             "    memory.page_size = page;\n    memory.allocation_granularity = page;\n  }\n#endif\n", 1)
    text = text.replace('#include "tge/memory/system_ram.hpp"',
                        '#include "tge/memory/system_ram.hpp"\n#if !defined(_WIN32)\n#include <unistd.h>\n#endif', 1)
    open(path, "w").write(text)


def gguf_string(text):
    raw = text.encode()
    return struct.pack("<Q", len(raw)) + raw


def write_gguf(path, config, weights):
    """float32 GGUF v3 with the reference's names; dims[0] = columns (in), dims[1] = rows (out)."""
    names = {"model.embed_tokens.weight": "token_embd.weight", "model.norm.weight": "output_norm.weight",
             "lm_head.weight": "output.weight"}
    per_layer = {"input_layernorm.weight": "attn_norm.weight", "post_attention_layernorm.weight": "ffn_norm.weight",
                 "self_attn.q_proj.weight": "attn_q.weight", "self_attn.q_proj.bias": "attn_q.bias",
                 "self_attn.k_proj.weight": "attn_k.weight", "self_attn.k_proj.bias": "attn_k.bias",
                 "self_attn.v_proj.weight": "attn_v.weight", "self_attn.v_proj.bias": "attn_v.bias",
                 "self_attn.o_proj.weight": "attn_output.weight", "mlp.gate_proj.weight": "ffn_gate.weight",
                 "mlp.up_proj.weight": "ffn_up.weight", "mlp.down_proj.weight": "ffn_down.weight"}
    tensors = []
    for name, value in weights.items():
        if name.startswith("model.layers."):
            _, _, index, rest = name.split(".", 3)
            out_name = f"blk.{index}.{per_layer[rest]}"
        else:
            out_name = names[name]
        tensors.append((out_name, np.ascontiguousarray(value.numpy().astype("<f4"))))
    heads = config["num_attention_heads"]
    kv = [("general.architecture", 8, "qwen2"),
          ("qwen2.block_count", 4, config["num_hidden_layers"]),
          ("qwen2.embedding_length", 4, config["hidden_size"]),
          ("qwen2.feed_forward_length", 4, config["intermediate_size"]),
          ("qwen2.attention.head_count", 4, heads),
          ("qwen2.attention.head_count_kv", 4, config.get("num_key_value_heads", heads)),
          ("qwen2.context_length", 4, config["max_position_embeddings"]),
          ("qwen2.attention.layer_norm_rms_epsilon", 6, config["rms_norm_eps"]),
          ("qwen2.rope.freq_base", 6, config["rope_theta"])]
    blob = struct.pack("<IIQQ", 0x46554747, 3, len(tensors), len(kv))
    for key, kind, value in kv:
        blob += gguf_string(key) + struct.pack("<I", kind)
        blob += gguf_string(value) if kind == 8 else struct.pack("<I" if kind == 4 else "<f", value)
    offset = 0
    for name, array in tensors:
        dims = list(reversed(array.shape))
        blob += gguf_string(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        blob += struct.pack("<IQ", 0, offset)
        offset += (array.nbytes + 31) // 32 * 32
    blob += b"\0" * ((32 - len(blob) % 32) % 32)
    with open(path, "wb") as handle:
        handle.write(blob)
        for _, array in tensors:
            handle.write(array.tobytes())
            handle.write(b"\0" * ((32 - array.nbytes % 32) % 32))


def weights_hash(weights):
    digest = hashlib.sha256()
    for name in sorted(weights):
        digest.update(name.encode())
        digest.update(weights[name].numpy().astype("<f4").tobytes())
    return digest.hexdigest()


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", required=True, help="checkout of the reference engine (read only)")
    args = parser.parse_args()
    import torch
    from aegean_tge_b200 import write_random_model
    from aegean_tge_b200.weights import ModelFiles
    from conftest import TINY
    work = tempfile.mkdtemp(prefix="tge_golden_")
    tree = os.path.join(work, "ref")
    shutil.copytree(args.reference, tree)
    subprocess.run(["chmod", "-R", "u+w", tree], check=True)
    shim(tree)
    build = os.path.join(tree, "build")
    subprocess.run(["cmake", "-S", tree, "-B", build, "-G", "Ninja", "-DCMAKE_BUILD_TYPE=Release",
                    "-DTGE_ENABLE_VULKAN=OFF", "-DTGE_BUILD_TESTS=OFF"], check=True, stdout=subprocess.DEVNULL)
    subprocess.run(["cmake", "--build", build], check=True, stdout=subprocess.DEVNULL)
    driver = os.path.join(work, "reference_driver")
    subprocess.run(["g++", "-std=c++20", "-O2", "-I", os.path.join(tree, "include"),
                    os.path.join(HERE, "reference_driver.cpp"), os.path.join(build, "lib", "libtge_core.a"),
                    "-lpthread", "-o", driver], check=True)
    for name in ("A", "B"):
        config, seed = TINY[name]
        folder = os.path.join(work, f"tiny_{name}")
        write_random_model(folder, config, seed=seed, dtype="float32")
        files = ModelFiles(folder)
        weights = {n: files.read(n).clone() for n in files.names()}
        gguf = os.path.join(work, f"tiny_{name}.gguf")
        write_gguf(gguf, config, weights)
        rnd = random.Random(100 + seed)
        vocab = config["vocab_size"]
        first = [rnd.randrange(vocab) for _ in range(21)]      # sequence 0: 17-token prompt + 4 decode steps
        second = [rnd.randrange(vocab) for _ in range(9)]      # sequence 1
        lines = ["prefill 0 17 " + " ".join(map(str, first[:17]))]
        rows = [("first", 16)]
        for step in range(17, 21):
            lines.append(f"forward 0 {first[step]} {step}")
            rows.append(("first", step))
        lines.append("batch 9 " + " ".join(f"{t} {p} 1" for p, t in enumerate(second)))    # all rows of sequence 1
        rows += [("second", p) for p in range(9)]
        # mixed: three more rows of sequence 1 would need its earlier rows cached: they are (positions 0..8)
        extra = [rnd.randrange(vocab) for _ in range(3)]
        more = rnd.randrange(vocab)
        lines.append("batch 4 " + " ".join(f"{t} {9 + i} 1" for i, t in enumerate(extra)) + f" {more} 21 0")
        rows += [("second", 9), ("second", 10), ("second", 11), ("first", 21)]
        script = os.path.join(work, f"script_{name}.txt")
        open(script, "w").write("\n".join(lines) + "\n")
        out = os.path.join(work, f"out_{name}.f32")
        subprocess.run([driver, gguf, script, out, "2"], check=True)
        logits = np.fromfile(out, dtype="<f4").reshape(-1, vocab)
        assert logits.shape[0] == len(rows)
        np.savez_compressed(os.path.join(HERE, f"tiny_{name}.npz"), logits=logits,
                            first=np.array(first + [more]), second=np.array(second + extra),
                            row_sequence=np.array([0 if r[0] == "first" else 1 for r in rows]),
                            row_position=np.array([r[1] for r in rows]), seed=np.array(seed),
                            weights_sha256=np.array(weights_hash(weights)), script=np.array("\n".join(lines)))
        print(f"tiny_{name}: {logits.shape[0]} rows written; weights {weights_hash(weights)[:16]}")
    make_sampler_golden(work, tree, build)
    shutil.rmtree(work)


def make_sampler_golden(work, tree, build):
    driver = os.path.join(work, "reference_sampler_driver")
    subprocess.run(["g++", "-std=c++20", "-O2", "-I", os.path.join(tree, "include"),
                    os.path.join(HERE, "reference_sampler_driver.cpp"), os.path.join(build, "lib", "libtge_core.a"),
                    "-lpthread", "-o", driver], check=True)
    vocab = 331
    rng = np.random.default_rng(77)
    logits = (rng.standard_normal((6, vocab)) * np.array([0.5, 1.0, 2.0, 4.0, 1.0, 3.0])[:, None]).astype("<f4")
    logits[4, [7, 90, 200]] = logits[4].max() + 1.0                 # a three-way tie at the top
    logits_path = os.path.join(work, "sampler_logits.f32")
    logits.tofile(logits_path)
    history = [int(t) for t in rng.integers(0, vocab, 40)] + [7, 7, 90]
    # row, draws, seed, temperature, top_k, top_p, min_p, repeat_penalty, penalty_window, history
    cases = [(0, 1, 0, 0.0, 0, 1.0, 0.0, 1.0, 64, []),              # greedy
             (4, 1, 0, 0.0, 0, 1.0, 0.0, 1.0, 64, []),              # greedy on a tie: the first index
             (4, 1, 0, 0.0, 0, 1.0, 0.0, 1.3, 0, history),          # greedy after the penalty moved the tie
             (1, 40, 0, 1.0, 0, 1.0, 0.0, 1.0, 64, []),             # temperature, the default seed
             (2, 40, 12345, 0.7, 0, 1.0, 0.0, 1.0, 64, []),
             (3, 40, 99, 1.5, 0, 1.0, 0.0, 1.0, 64, []),
             (1, 40, 5, 1.0, 5, 1.0, 0.0, 1.0, 64, []),             # top-k
             (2, 40, 6, 0.9, 0, 0.8, 0.0, 1.0, 64, []),             # top-p
             (3, 40, 7, 1.2, 0, 1.0, 0.05, 1.0, 64, []),            # min-p
             (5, 40, 8, 1.0, 50, 0.9, 0.02, 1.0, 64, []),           # all three cuts
             (1, 40, 9, 1.0, 0, 1.0, 0.0, 1.5, 16, history),        # penalty over a window
             (5, 40, 10, 0.8, 20, 0.95, 0.0, 1.2, 0, history)]      # cuts and penalty over the whole history
    lines = [" ".join(str(x) for x in case[:9]) + f" {len(case[9])} " + " ".join(map(str, case[9])) for case in cases]
    cases_path = os.path.join(work, "sampler_cases.txt")
    open(cases_path, "w").write("\n".join(lines) + "\n")
    out = subprocess.run([driver, logits_path, str(vocab), cases_path], check=True, capture_output=True, text=True).stdout
    picks = [[int(t) for t in line.split()] for line in out.strip().splitlines()]
    assert [len(p) for p in picks] == [case[1] for case in cases]
    np.savez_compressed(os.path.join(HERE, "sampler.npz"), logits=logits, cases=np.array(lines),
                        picks=np.array([p + [-1] * (40 - len(p)) for p in picks]))
    print(f"sampler: {sum(len(p) for p in picks)} draws written")


if __name__ == "__main__":
    main()
