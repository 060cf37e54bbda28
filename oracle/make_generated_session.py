"""Generates buddy-mlir's ModelSession for the small test model with the reference's own
generators, for oracle/session_host.cpp (test infrastructure; see there).

    python oracle/make_generated_session.py <buddy-mlir root> <output dir>

Runs tools/buddy-codegen/gen_config.py (variant spec + HuggingFace-style config -> full
model config) and tools/buddy-codegen/gen_session.py (config -> ModelSession.h / .cpp) as
they stand, once per flavour, and writes their output to <output dir>/<flavour>/
(oracle/_ref/generated, which is not committed: it is generated reference code).  The model is
TINY_QWEN2 of buddy_mlir_b200/config.py; the flavours are the seven variants of
gen_config.py:37-71 plus the tiered-cache and the packed-decode spec of
models/deepseek_r1/specs/ (f32 both), with the small model's sizes in place of the 1.5B ones.
Prints the flavour names, one per line."""
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

FLAVOURS = ("f32", "f16", "bf16", "w8a32", "w8a8", "w8a16", "w4a16", "f32_tiered", "f32_packed")


def spec_for(flavour, cfg, synthetic):
    from buddy_mlir_b200.gen_model_entry import TINY_TIERS
    variant = flavour.split("_")[0]
    total = synthetic.blob_elements(cfg)
    quantised = sum(int(s[0] * s[1]) for n, _, s in synthetic.tensor_list(cfg) if n in synthetic.QUANTISED_BY_REFERENCE)
    scales = sum(int(s[1]) for n, _, s in synthetic.tensor_list(cfg) if n in synthetic.QUANTISED_BY_REFERENCE)
    spec = {"hf_model_path": "local/tiny_qwen2", "model_family": "deepseek_r1", "variant": variant,
            "max_token_len": cfg.max_len, "num_threads": 8,
            "weights_override": {"total": total, "linear_elements": 0, "linear_output_channels": 0, "other_elements": 0}}
    if variant.startswith("w"):
        # the float file holds the unquantised tensors and one scale per quantised column
        # (gen_config.py:207-247: other_elements + linear_output_channels); the int file the
        # quantised elements, two per byte for int4
        spec["quantization"] = variant
        spec["weights_override"] = {"total": total, "linear_elements": quantised // (2 if variant == "w4a16" else 1),
                                    "linear_output_channels": scales, "other_elements": total - quantised}
    if flavour == "f32_tiered":
        spec["tiered_kv_cache"] = {"enabled": True, "cache_sizes": list(TINY_TIERS)}
    if flavour == "f32_packed":
        spec["decode_pack_vector_size"] = 32
    return spec


def main(ref, out):
    sys.path.insert(0, os.path.join(ref, "tools", "buddy-codegen"))
    import gen_config
    import gen_session
    from buddy_mlir_b200 import TINY_QWEN2 as cfg, synthetic
    os.makedirs(out, exist_ok=True)
    hf = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_size": cfg.hidden,
          "intermediate_size": cfg.ffn, "num_hidden_layers": cfg.n_layers, "num_attention_heads": cfg.q_heads,
          "num_key_value_heads": cfg.kv_heads, "vocab_size": cfg.vocab, "max_position_embeddings": cfg.max_len,
          "rms_norm_eps": cfg.eps, "rope_theta": cfg.rope_theta, "head_dim": cfg.head_dim, "eos_token_id": cfg.vocab - 1,
          "bos_token_id": 1, "tie_word_embeddings": False}
    hf_path = os.path.join(out, "hf_config.json")
    with open(hf_path, "w") as f:
        json.dump(hf, f)
    for flavour in FLAVOURS:
        d = os.path.join(out, flavour)
        os.makedirs(os.path.join(d, "buddy", "runtime", "models"), exist_ok=True)
        config = gen_config.gen_config(spec_for(flavour, cfg, synthetic), hf_path)
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(config, f, indent=1)
        with open(os.path.join(d, "buddy", "runtime", "models", "ModelSession.h"), "w") as f:
            f.write(gen_session.gen_header(config))
        with open(os.path.join(d, "ModelSession.cpp"), "w") as f:
            f.write(gen_session.gen_impl(config))
        print(flavour)


if __name__ == "__main__":
    main(sys.argv[1], sys.argv[2])
