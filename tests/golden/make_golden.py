"""Writes tests/golden/tiny_{a,b}.npz from the reference project's own second implementation.

Run once, on a machine that has the reference's sources (its pure-NumPy `etalii_dllm.reference` imports without the
native extension):

    python tests/golden/make_golden.py /path/to/reference/src

For the two tiny Llama configurations of tests/plain_llama.py it stores, per prompt, the logits after every prompt
token (fed one at a time through `ReferenceTransformer.forward`) and the tokens of a greedy and of a seeded
temperature-0.8 generation (`ReferenceTransformer.generate` with `reference.Sampler`). tests/test_plain.py compares
the plain implementation with these files; nothing else reads the reference.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import plain_llama as P  # noqa: E402

PROMPT_LENGTHS = {"a": (5, 11, 17), "b": (1, 7, 23, 40)}
STD = {"a": 0.02, "b": 0.08}
"""Tiny B uses wider weights so that attention scores and the sampled tokens really depend on the keys."""


def reference_names(config, weights):
    """Hugging Face names -> the reference's internal names (src/etalii_dllm/importing/importer.py:74-113)."""
    layer = {
        "input_layernorm.weight": "attention_norm.weight", "self_attn.q_proj.weight": "attention.q.weight",
        "self_attn.k_proj.weight": "attention.k.weight", "self_attn.v_proj.weight": "attention.v.weight",
        "self_attn.o_proj.weight": "attention.o.weight", "post_attention_layernorm.weight": "mlp_norm.weight",
        "mlp.gate_proj.weight": "mlp.gate.weight", "mlp.up_proj.weight": "mlp.up.weight",
        "mlp.down_proj.weight": "mlp.down.weight",
    }
    out = {}
    for name, value in weights.items():
        if name == "model.embed_tokens.weight":
            out["token_embedding.weight"] = value
        elif name == "model.norm.weight":
            out["final_norm.weight"] = value
        elif name == "lm_head.weight":
            out[name] = value
        else:
            _, _, index, rest = name.split(".", 3)
            out[f"layers.{index}.{layer[rest]}"] = value
    return out


def main(reference_src: str) -> None:
    sys.path.insert(0, reference_src)
    import etalii_dllm.reference as ref
    from etalii_dllm.architecture import TransformerConfig

    for tag, config, seed in (("a", P.TINY_A, 0), ("b", P.TINY_B, 1)):
        eos = config["eos_token_id"]
        cfg = TransformerConfig(
            family="llama", vocabulary_size=config["vocab_size"], hidden_size=config["hidden_size"],
            intermediate_size=config["intermediate_size"], layers=config["num_hidden_layers"],
            heads=config["num_attention_heads"], kv_heads=config["num_key_value_heads"], head_dim=config["head_dim"],
            context_length=config["max_position_embeddings"], rms_norm_eps=config["rms_norm_eps"],
            rope_theta=config["rope_theta"], rope_scaling=config.get("rope_scaling"),
            tie_word_embeddings=config["tie_word_embeddings"],
            eos_token_ids=tuple(eos) if isinstance(eos, list) else (eos,),
        )
        weights = P.random_weights(config, seed, std=STD[tag])
        model = ref.ReferenceTransformer(cfg, reference_names(config, weights))
        rng = np.random.default_rng(100 + seed)
        out = {}
        for index, length in enumerate(PROMPT_LENGTHS[tag]):
            prompt = rng.integers(0, config["vocab_size"], length).tolist()
            model.reset()
            logits = np.stack([model.forward([t]) for t in prompt])
            greedy, _ = model.generate(prompt, 8, ref.Sampler(0.0), stop_tokens=())
            sampled, _ = model.generate(prompt, 12, ref.Sampler(0.8, 0, 1.0, seed=seed + index), stop_tokens=())
            nucleus, _ = model.generate(prompt, 12, ref.Sampler(1.3, 20, 0.9, seed=7 + index, min_p=0.02),
                                        stop_tokens=())
            out[f"prompt{index}"] = np.array(prompt, np.int32)
            out[f"logits{index}"] = logits.astype(np.float32)
            out[f"greedy{index}"] = np.array(greedy, np.int32)
            out[f"sampled{index}"] = np.array(sampled, np.int32)
            out[f"nucleus{index}"] = np.array(nucleus, np.int32)
        out["inv_freq"] = model.inv_freq
        np.savez_compressed(os.path.join(HERE, f"tiny_{tag}.npz"), **out)
        print(tag, "written")


if __name__ == "__main__":
    main(sys.argv[1])
