"""Generates buddy-mlir's ModelSession for the small test model with the reference's own
generators, for oracle/session_host.cpp (test infrastructure; see there).

    python oracle/make_generated_session.py <buddy-mlir root> <output dir>

Runs tools/buddy-codegen/gen_config.py (variant spec + HuggingFace-style config -> full
model config) and tools/buddy-codegen/gen_session.py (config -> ModelSession.h / .cpp) as
they stand and writes their output under <output dir> (oracle/_ref/generated, which is not
committed: it is generated reference code).  The model is TINY_QWEN2 of
buddy_mlir_b200/config.py, variant f32."""
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))


def main(ref, out):
    sys.path.insert(0, os.path.join(ref, "tools", "buddy-codegen"))
    import gen_config
    import gen_session
    from buddy_mlir_b200 import TINY_QWEN2 as cfg, synthetic
    os.makedirs(os.path.join(out, "buddy", "runtime", "models"), exist_ok=True)
    hf = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_size": cfg.hidden,
          "intermediate_size": cfg.ffn, "num_hidden_layers": cfg.n_layers, "num_attention_heads": cfg.q_heads,
          "num_key_value_heads": cfg.kv_heads, "vocab_size": cfg.vocab, "max_position_embeddings": cfg.max_len,
          "rms_norm_eps": cfg.eps, "rope_theta": cfg.rope_theta, "head_dim": cfg.head_dim, "eos_token_id": cfg.vocab - 1,
          "bos_token_id": 1, "tie_word_embeddings": False}
    hf_path = os.path.join(out, "hf_config.json")
    with open(hf_path, "w") as f:
        json.dump(hf, f)
    spec = {"hf_model_path": "local/tiny_qwen2", "model_family": "deepseek_r1", "variant": "f32",
            "max_token_len": cfg.max_len, "num_threads": 8,
            "weights_override": {"total": synthetic.blob_elements(cfg), "linear_elements": 0,
                                 "linear_output_channels": 0, "other_elements": 0}}
    config = gen_config.gen_config(spec, hf_path)
    with open(os.path.join(out, "config.json"), "w") as f:
        json.dump(config, f, indent=1)
    with open(os.path.join(out, "buddy", "runtime", "models", "ModelSession.h"), "w") as f:
        f.write(gen_session.gen_header(config))
    with open(os.path.join(out, "ModelSession.cpp"), "w") as f:
        f.write(gen_session.gen_impl(config))


if __name__ == "__main__":
    main(sys.argv[1], sys.argv[2])
