"""Runs buddy-mlir's own importer (tools/buddy-codegen/import_model.py) on the small Qwen2
model and records what it writes into the weight files, so that the blob walk of this
library (synthetic.tensor_list, b200_model_load_blobs) is pinned to the reference's code
and not to a reading of it.  Run from the repo root, with a buddy-mlir checkout:

    BUDDY_MLIR_ROOT=<buddy-mlir> python tests/golden/make_reference_blobs.py

The importer is used as it stands: compile_graphs (TorchDynamo trace of the HuggingFace
module through DynamoCompiler), apply_pre_transforms (weights become [K,N]),
apply_quantization, extract_plain_weights / extract_quantized_weights.  Only the MLIR Python
bindings, which those steps import but do not call, are replaced by empty modules.  The
weights are the seeded tensors of synthetic.make_f32_blob loaded into
transformers.Qwen2ForCausalLM.

Output: reference_importer_tiny_qwen2.npz
  order            the parameters in the importer's order, as "<tensor>:<layer>" names found
                   by comparing contents with the seeded tensors
  quantised        the names the quantisation pass turned into int8
  <variant>_<bucket>_sha256, _size   digest and element count of every bucket the importer
                   returns (f32 / f16 / bf16: params, and for f32 decode_packed, the decode file of
                   the packed-decode spec; w8a32 / w8a8: f32_params, i8_params; w8a16: f16_params,
                   i8_params; w4a16: f16_params, i4_params)
  w8a32_scales     the scale section at the end of the w8a32 float bucket
  inv_freq         the rotary buffer as the HuggingFace module computed it (the one tensor that
                   is not loaded from the seeded weights)
  w8a8_prefill_ops, w8a8_decode_ops
                   "<operation>:<weight>:<activation shape>" of every integer matmul the w8a8 pass
                   left in the two graphs
  qwen3_order      the same order for the small Qwen3 model (head norms, no biases)
  prefill_inputs, prefill_outputs, decode_inputs, decode_outputs
                   "<shape>:<dtype>" of the traced graphs' inputs (after the parameters) and, with the
                   producing operation, of their outputs: the entry ABI of the compiled model
"""
import hashlib
import importlib.abc
import importlib.machinery
import importlib.util
import os
import sys
import types
from unittest import mock

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = os.environ.get("BUDDY_MLIR_ROOT") or os.path.join(os.path.dirname(ROOT), "reference")
sys.path.insert(0, ROOT)

from buddy_mlir_b200 import TINY_QWEN2, synthetic  # noqa: E402

SEED_W = 1234


class _NoBindings(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def find_spec(self, name, path, target=None):
        if name == "buddy_mlir" or name.startswith("buddy_mlir."):
            return importlib.machinery.ModuleSpec(name, self, is_package=True)
        return None

    def create_module(self, spec):
        m = mock.MagicMock(name=spec.name)
        m.__path__, m.__name__, m.__spec__ = [], spec.name, spec
        return m

    def exec_module(self, module):
        pass


def load_importer():
    sys.meta_path.insert(0, _NoBindings())
    top, comp = types.ModuleType("buddy"), types.ModuleType("buddy.compiler")
    top.__path__, comp.__path__ = [], [os.path.join(REF, "frontend", "Python")]
    top.compiler = comp
    sys.modules["buddy"], sys.modules["buddy.compiler"] = top, comp
    spec = importlib.util.spec_from_file_location(
        "reference_import_model", os.path.join(REF, "tools", "buddy-codegen", "import_model.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def hf_model(cfg, views, act):
    import torch
    import transformers
    common = dict(
        hidden_size=cfg.hidden, intermediate_size=cfg.ffn, num_hidden_layers=cfg.n_layers,
        num_attention_heads=cfg.q_heads, num_key_value_heads=cfg.kv_heads, vocab_size=cfg.vocab,
        max_position_embeddings=cfg.max_len, rms_norm_eps=cfg.eps, rope_theta=cfg.rope_theta,
        tie_word_embeddings=False, head_dim=cfg.head_dim)
    if cfg.qk_norm:
        model = transformers.Qwen3ForCausalLM(transformers.Qwen3Config(**common, attention_bias=False))
    else:
        model = transformers.Qwen2ForCausalLM(transformers.Qwen2Config(**common))
    model = model.float().eval()
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a))   # noqa: E731
    sd = {"model.embed_tokens.weight": t(views[("embed", -1)]), "model.norm.weight": t(views[("final_norm", -1)]),
          "lm_head.weight": t(views[("lm_head", -1)].T)}
    for l in range(cfg.n_layers):
        p = f"model.layers.{l}."
        sd[p + "input_layernorm.weight"] = t(views[("in_norm", l)])
        sd[p + "post_attention_layernorm.weight"] = t(views[("post_norm", l)])
        for n in ("q", "k", "v", "o"):
            sd[p + f"self_attn.{n}_proj.weight"] = t(views[(n, l)].T)
        if cfg.qkv_bias:
            for n in ("q", "k", "v"):
                sd[p + f"self_attn.{n}_proj.bias"] = t(views[(f"{n}_bias", l)])
        if cfg.qk_norm:
            sd[p + "self_attn.q_norm.weight"] = t(views[("q_norm", l)])
            sd[p + "self_attn.k_norm.weight"] = t(views[("k_norm", l)])
        for n in ("gate", "up", "down"):
            sd[p + f"mlp.{n}_proj.weight"] = t(views[(n, l)].T)
    missing, unexpected = model.load_state_dict(sd, strict=False)
    assert not unexpected and all("rotary" in m or "inv_freq" in m for m in missing), (missing, unexpected)
    if act == "f16":               # load_model, import_model.py:118-145
        model = model.half()
    elif act == "bf16":
        model = model.bfloat16()
    model.config.use_cache = False
    return model


def name_of(arr, views):
    for (name, layer), v in views.items():
        for cand in (v, v.T if v.ndim == 2 else None):
            if cand is not None and cand.shape == arr.shape and np.array_equal(cand.astype(arr.dtype), arr):
                return f"{name}:{layer}"
    # the rotary buffer is computed by the HuggingFace module itself, not loaded
    inv = views[("inv_freq", -1)]
    if arr.shape == inv.shape and np.allclose(arr, inv, rtol=1e-6, atol=0):
        return "inv_freq:-1"
    return "?"


def signature(node):
    dtype = str(node.tensor_meta["dtype"]).split(".")[-1].lower()
    return "x".join(str(int(s)) for s in node.tensor_meta["shape"]) + ":" + dtype


def digest(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def main():
    imp = load_importer()
    cfg = TINY_QWEN2
    _, views = synthetic.make_f32_blob(cfg, SEED_W)
    out = {"seed_w": SEED_W}
    activation = {"f32": "f32", "f16": "f16", "bf16": "bf16", "w8a32": "f32", "w8a8": "f32", "w8a16": "f16",
                  "w4a16": "f16"}
    for variant, act in activation.items():
        config = {"shape": {"max_token_len": cfg.max_len}, "variant": variant, "precision": {"activation_type": act}}
        model = hf_model(cfg, views, act)
        gp, gd, params = imp.compile_graphs(model, config)
        imp.apply_pre_transforms(gp[0], gd[0])
        if variant in ("f32", "f16", "bf16"):
            buckets = imp.extract_plain_weights(params, config)
        else:
            imp.apply_quantization(gp[0], gd[0], variant)
            buckets = imp.extract_quantized_weights(gp[0], params, config)
        if variant == "f32":
            out["order"] = np.array([name_of(p.detach().numpy(), views) for p in params])
            assert "?" not in out["order"], out["order"]
            out["inv_freq"] = params[list(out["order"]).index("inv_freq:-1")].detach().numpy().copy()
            # the signatures of the two traced graphs: what _mlir_ciface_forward_prefill / _decode
            # receive after the weight blobs, and what their result structs hold
            for phase, g in (("prefill", gp[0]), ("decode", gd[0])):
                out[f"{phase}_inputs"] = np.array([signature(n) for n in g.inputs])
                ret = [n for n in g.body if type(n).__name__ == "OutputOp"][0]
                out[f"{phase}_outputs"] = np.array([signature(g.node_table[a]) + ":" + type(g.node_table[a]).__name__
                                                    for a in ret.args])
                print(phase, "inputs", list(out[f"{phase}_inputs"]), "outputs", list(out[f"{phase}_outputs"]))
            # the decode file of the packed-decode spec: the decode graph's own parameter list after
            # pack_decode_matmul_weights (import_model.py:463-481, 1214-1226)
            imp.pack_decode_weights(gd[0], {"vector_size": 32})
            buckets["decode_packed"] = np.concatenate([p.detach().numpy().reshape(-1) for p in gd[0]._params_ref])
        if variant == "w8a32":
            from buddy.compiler.graph.type import TensorDType
            names = [name_of(p.detach().numpy(), views) for p in params]
            out["quantised"] = np.array([n for n, node in zip(names, gp[0].params)
                                         if node.tensor_meta.get("dtype") == TensorDType.Int8])
            n_scales = sum(int(np.prod(node.tensor_meta["shape"])) for node in gp[0].params[len(params):])
            out["w8a32_scales"] = buckets["f32_params"][-n_scales:].copy()
        if variant == "w8a8":
            # which projections the w8a8 pass turned into integer matmuls, and the activation tensor
            # each of them quantises as a whole (its shape: all rows of the prefill, one row of a decode)
            for phase, g in (("prefill", gp[0]), ("decode", gd[0])):
                # both graphs were traced from the same module: the same parameters in the same order
                assert all(list(node.tensor_meta["shape"]) == list(p.shape) for node, p in zip(g.params, params))
                names = {node.name: name_of(p.detach().numpy(), views) for node, p in zip(g.params, params)}
                rows = []
                for node in g.body:
                    kind = type(node).__name__
                    if kind in ("QuantizedMatmulOp", "QuantizedAddMMOp"):
                        act, weight = (node.args[0], node.args[1]) if kind == "QuantizedMatmulOp" else (node.args[1], node.args[2])
                        shape = "x".join(str(int(s)) for s in g.node_table[act].tensor_meta["shape"])
                        rows.append(f"{kind}:{names.get(weight, weight)}:{shape}")
                out[f"w8a8_{phase}_ops"] = np.array(rows)
                print("w8a8", phase, rows)
        for tag, arr in buckets.items():
            out[f"{variant}_{tag}_sha256"] = digest(arr)
            out[f"{variant}_{tag}_size"] = arr.size
            out[f"{variant}_{tag}_dtype"] = str(arr.dtype)
            print(f"{variant}: {tag} {arr.dtype} x {arr.size}")
    # Qwen3 (head norms, no biases): the parameter order only
    from buddy_mlir_b200 import TINY_QWEN3
    _, views3 = synthetic.make_f32_blob(TINY_QWEN3, SEED_W)
    config = {"shape": {"max_token_len": TINY_QWEN3.max_len}, "variant": "f32", "precision": {"activation_type": "f32"}}
    _, _, params3 = imp.compile_graphs(hf_model(TINY_QWEN3, views3, "f32"), config)
    out["qwen3_order"] = np.array([name_of(p.detach().numpy(), views3) for p in params3])
    assert "?" not in out["qwen3_order"], out["qwen3_order"]
    print("qwen3 order:", list(out["qwen3_order"]))
    path = os.path.join(HERE, "reference_importer_tiny_qwen2.npz")
    np.savez_compressed(path, **out)
    print("order:", list(out["order"]))
    print("written", path)


if __name__ == "__main__":
    main()
