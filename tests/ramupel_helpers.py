"""Small Ramupel configurations with sizes of their own, and seeded model folders for them."""
import json
import os

import torch

# Odd sizes: heads of unequal shapes, a layer without a feed-forward, a rotation over part of the rotated
# dimensions, one head, more value columns than one CTA of the recurrence takes, head outputs whose width is no
# multiple of 8 (those products leave the tensor cores).
SMALL = {
    "architecture": "Ramupel", "vocab": 203, "width": 88, "embedding": {"scale": 2.5}, "norm": {"eps": 3e-6},
    "layers": [
        {"type": "latent_attention", "mlp": {"kind": "dense", "ff": 136},
         "mixer": {"heads": 3, "dim": 24, "rot_dim": 12, "vdim": 20, "kv_rank": 40, "scale": 0.2,
                   "rot": {"base": 10000.0, "dims": 8}}},
        {"type": "gla", "mlp": None, "mixer": {"heads": 2, "dim": 20, "vdim": 36, "tau": 8.0}},
        {"type": "latent_attention", "mlp": {"kind": "dense", "ff": 200},
         "mixer": {"heads": 1, "dim": 16, "rot_dim": 4, "vdim": 48, "kv_rank": 72, "scale": 0.25,
                   "rot": {"base": 500.0, "dims": 4}}},
        {"type": "gla", "mlp": {"kind": "dense", "ff": 64}, "mixer": {"heads": 3, "dim": 6, "vdim": 70, "tau": 3.0}},
    ],
}
# Sizes the tensor-core products take; more heads than one CTA of the latent attention has rows.
WIDE = {
    "architecture": "Ramupel", "vocab": 320, "width": 128, "embedding": {"scale": 11.3}, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "gla", "mlp": {"kind": "dense", "ff": 256}, "mixer": {"heads": 2, "dim": 64, "vdim": 128, "tau": 16.0}},
        {"type": "latent_attention", "mlp": {"kind": "dense", "ff": 192},
         "mixer": {"heads": 4, "dim": 64, "rot_dim": 32, "vdim": 64, "kv_rank": 160, "scale": 0.1,
                   "rot": {"base": 1000000.0, "dims": 32}}},
        {"type": "latent_attention", "mlp": {"kind": "dense", "ff": 128},
         "mixer": {"heads": 40, "dim": 8, "rot_dim": 8, "vdim": 8, "kv_rank": 24, "scale": 0.25,
                   "rot": {"base": 10000.0, "dims": 8}}},
    ],
}
# A width that is no multiple of 8 (every product leaves the tensor cores, also in bfloat16), a latent rank that is
# no multiple of 8 and values wider than the padded key (so prompts keep the absorbed form), 130 key channels.
RAGGED = {
    "architecture": "Ramupel", "vocab": 131, "width": 92, "embedding": {"scale": 0.7}, "norm": {"eps": 2e-5},
    "layers": [
        {"type": "gla", "mlp": {"kind": "dense", "ff": 50}, "mixer": {"heads": 1, "dim": 130, "vdim": 16, "tau": 5.0}},
        {"type": "latent_attention", "mlp": None,
         "mixer": {"heads": 2, "dim": 8, "rot_dim": 6, "vdim": 80, "kv_rank": 36, "scale": 0.3,
                   "rot": {"base": 100.0, "dims": 6}}},
        {"type": "latent_attention", "mlp": {"kind": "dense", "ff": 92},
         "mixer": {"heads": 5, "dim": 10, "rot_dim": 6, "vdim": 12, "kv_rank": 52, "scale": 0.25,
                   "rot": {"base": 10000.0, "dims": 6}}},
    ],
}
CONFIGS = {"small": (SMALL, 11, 0.09, (5, 24)), "wide": (WIDE, 12, 0.05, (8,)), "ragged": (RAGGED, 13, 0.08, (3,))}

# bfloat16: at most four times the worst error the comparisons of each configuration achieved on a B200
BFLOAT16_BOUND = {"small": 4e-2, "wide": 4e-2, "ragged": 4e-2}


def bound(dtype, name):
    return 2e-5 if dtype == "float32" else BFLOAT16_BOUND[name]


def make_model(tmp_path, name, dtype="bfloat16"):
    """A model folder for configuration ``name``: the library's seeded writer, then the tensors whose random
    draw around zero would switch a mechanism off (depth weights, decay biases, activation numbers, gate biases)
    and the decay factors (whose width the file decides) are drawn again here."""
    from llmplayer_b200.config import config_from_dict
    from llmplayer_b200.weights import write_random_model
    from llmplayer_b200.weights.safetensors_io import write_safetensors
    from plain_llama import read_safetensors
    raw, seed, std, ranks = CONFIGS[name]
    out = os.path.join(str(tmp_path), f"ramupel_{name}_{dtype}")
    write_random_model(config_from_dict(raw), seed, out, dtype=dtype, std=std)
    path = os.path.join(out, "model.safetensors")
    tensors = read_safetensors(path)
    gen = torch.Generator().manual_seed(seed + 100)
    store = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    gla_seen = 0
    for i, layer in enumerate(raw["layers"]):
        p = f"l{i}."
        signs = torch.where(torch.rand(i + 2, generator=gen) < 0.3, -1.0, 1.0)
        tensors[p + "dwa"] = ((0.3 + 0.6 * torch.rand(i + 2, generator=gen)) * signs).to(store)
        tensors[p + "rg1.b"] = (0.7 * torch.randn(raw["width"], generator=gen)).to(store)
        if layer["mlp"] is not None:
            tensors[p + "rg2.b"] = (0.7 * torch.randn(raw["width"], generator=gen)).to(store)
            tensors[p + "mlp.act"] = torch.randn(2, generator=gen).to(store)
        if layer["type"] == "gla":
            m = layer["mixer"]
            rank = ranks[gla_seen % len(ranks)]
            gla_seen += 1
            tensors[p + "mix.a1"] = (0.3 * torch.randn(rank, raw["width"], generator=gen)).to(store)
            tensors[p + "mix.a2"] = (0.5 * torch.randn(m["heads"] * m["dim"], rank, generator=gen)).to(store)
            tensors[p + "mix.a2.b"] = (2.0 + 2.0 * torch.randn(m["heads"] * m["dim"], generator=gen)).to(store)
    write_safetensors(path, tensors, metadata={"format": "pt"})
    with open(os.path.join(out, "config.json"), "w") as fh:
        json.dump(raw, fh, indent=1)
    return out


def plain_logits(model_dir, tokens, rows=None):
    import plain_ramupel
    cfg, w = plain_ramupel.read_model(model_dir)
    return plain_ramupel.forward(cfg, w, tokens, dtype=torch.float64, rows=rows)
