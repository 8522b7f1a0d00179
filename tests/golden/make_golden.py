"""Runs nesmind/matricxon's own StarCoder2 model code on the CPU for the two tiny test
configurations and stores its logits beside this script.

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/reference

The reference tree is put on sys.path (read-only use); our seeded tensors are written as an
F32 GGUF with the reference's own builder (tools/make_tiny_gguf.py:24-116) under the GGUF
names its loader expects (app/architectures/starcoder2.py:133-194), then loaded and run
through ``Starcoder2Architecture.from_gguf`` (app/architectures/starcoder2.py:112-127) in
float32 without a cache. Limits of the anchor: the reference has no sliding window, so
prompts are shorter than the window; it has a bias on every projection, so the
configuration without biases is given zero biases.
"""

import os
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
sys.path.insert(0, str(HERE.parent.parent))

PROMPT_LENGTHS = {"A": 24, "B": 20}     # below the windows (32 and 24)

GGUF_NAMES = {
    "model.embed_tokens.weight": "token_embd.weight",
    "model.norm.weight": "output_norm.weight",
    "model.norm.bias": "output_norm.bias",
    "lm_head.weight": "output.weight",
}
LAYER_NAMES = {
    "input_layernorm": "attn_norm", "post_attention_layernorm": "ffn_norm",
    "self_attn.q_proj": "attn_q", "self_attn.k_proj": "attn_k", "self_attn.v_proj": "attn_v",
    "self_attn.o_proj": "attn_output", "mlp.c_fc": "ffn_up", "mlp.c_proj": "ffn_down",
}


def gguf_name(name: str) -> str:
    if name in GGUF_NAMES:
        return GGUF_NAMES[name]
    _, _, index, rest = name.split(".", 3)
    module, kind = rest.rsplit(".", 1)
    return f"blk.{index}.{LAYER_NAMES[module]}.{kind}"


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path to a checkout of nesmind/matricxon>")
    reference = sys.argv[1]
    sys.path.insert(0, reference)
    from app.architectures.starcoder2 import Starcoder2Architecture
    from app.gguf.constants import GGMLQuantizationType
    from app.gguf.loader import GGUFModelLoader
    from tools.make_tiny_gguf import GGUFBuilder

    from tiny_configs import TINY, random_ids, tiny_tensors

    for name, (raw, _, _) in TINY.items():
        tensors = tiny_tensors(name)
        builder = (GGUFBuilder()
                   .set_str("general.architecture", "starcoder2")
                   .set_u32("starcoder2.embedding_length", raw["hidden_size"])
                   .set_u32("starcoder2.attention.head_count", raw["num_attention_heads"])
                   .set_u32("starcoder2.attention.head_count_kv", raw["num_key_value_heads"])
                   .set_u32("starcoder2.attention.key_length", raw["head_dim"])
                   .set_u32("starcoder2.block_count", raw["num_hidden_layers"])
                   .set_u32("starcoder2.feed_forward_length", raw["intermediate_size"])
                   .set_f32("starcoder2.attention.layer_norm_epsilon", raw["norm_epsilon"])
                   .set_u32("starcoder2.vocab_size", raw["vocab_size"])
                   .set_f32("starcoder2.rope.freq_base", raw["rope_theta"]))
        written = set()
        for hf_name, tensor in tensors.items():
            array = tensor.float().numpy().astype("<f4")
            target = gguf_name(hf_name)
            builder.add_tensor(target, list(reversed(array.shape)), GGMLQuantizationType.F32,
                               array.tobytes())
            written.add(target)
        if not raw["use_bias"]:
            # the reference requires a bias on every projection: zeros leave the maths unchanged
            shapes = {"attn_q": raw["num_attention_heads"] * raw["head_dim"],
                      "attn_k": raw["num_key_value_heads"] * raw["head_dim"],
                      "attn_v": raw["num_key_value_heads"] * raw["head_dim"],
                      "attn_output": raw["hidden_size"], "ffn_up": raw["intermediate_size"],
                      "ffn_down": raw["hidden_size"]}
            for layer in range(raw["num_hidden_layers"]):
                for module, size in shapes.items():
                    builder.add_tensor(f"blk.{layer}.{module}.bias", [size],
                                       GGMLQuantizationType.F32, np.zeros(size, "<f4").tobytes())
        with tempfile.TemporaryDirectory() as tmp:
            path = builder.write(Path(tmp) / f"tiny_{name}.gguf")
            loader = GGUFModelLoader(str(path), dtype=torch.float32)
            model = Starcoder2Architecture.from_gguf(loader, dtype=torch.float32).eval()
            ids = random_ids(PROMPT_LENGTHS[name], raw["vocab_size"], seed=100 + ord(name))
            with torch.no_grad():
                logits = model(torch.tensor([ids], dtype=torch.long))[0]
        np.save(HERE / f"reference_logits_{name}.npy", logits.float().numpy())
        print(name, "prompt", len(ids), "logits", tuple(logits.shape),
              "max|logit|", float(logits.abs().max()))


if __name__ == "__main__":
    os.environ.setdefault("PYTHONDONTWRITEBYTECODE", "1")
    main()
