#!/usr/bin/env python3
"""Builds tests/golden/bert_tiny_golden.npz and tests/golden/bert_hf_seeded.npz.

1. bert_tiny_golden.npz repacks Eos's committed known-answer fixture
   runtime/testdata/pretrained_bert_golden/{config.json,model.safetensors,golden.json}
   (tiny HF BertModel: hidden 16, 2 layers, 4 heads, FFN 32, vocab 17, max_len 12; expected
   masked-mean + L2 embeddings computed by PyTorch/transformers) into one numpy archive:
   the weights in the 16-tensors-per-layer order of runtime/pretrained_bert_importer.go:936-951,
   the three input id tensors, and the expected embeddings.  Tolerance of the Eos test that
   consumes it: max_abs <= 2e-3, min_cosine >= 0.9999
   (runtime/pretrained_bert_golden_parity_test.go:99-103).

2. bert_hf_seeded.npz is a second, larger seeded case made the same way the Eos fixture was
   (generate_fixture.py: a from-scratch transformers BertModel with uniform(-0.2, 0.2)
   weights), with ragged lengths: hidden 64, 3 layers, 4 heads, FFN 128, vocab 50, T=24, B=5.

Usage (needs the Eos checkout, torch, transformers, safetensors; run once, outputs are committed):
    python tests/golden/make_bert_golden_fixture.py /path/to/eos
"""
import json
import os
import sys

import numpy as np

LAYER_ORDER = [
    "attention.self.query.weight", "attention.self.query.bias",
    "attention.self.key.weight", "attention.self.key.bias",
    "attention.self.value.weight", "attention.self.value.bias",
    "attention.output.dense.weight", "attention.output.dense.bias",
    "attention.output.LayerNorm.weight", "attention.output.LayerNorm.bias",
    "intermediate.dense.weight", "intermediate.dense.bias",
    "output.dense.weight", "output.dense.bias",
    "output.LayerNorm.weight", "output.LayerNorm.bias",
]


def pack_state(state, layers):
    def get(name):
        for prefix in ("", "bert."):
            if prefix + name in state:
                return np.asarray(state[prefix + name], dtype=np.float32)
        raise KeyError(name)

    out = {
        "tok": get("embeddings.word_embeddings.weight"),
        "pos": get("embeddings.position_embeddings.weight"),
        "typ": get("embeddings.token_type_embeddings.weight"),
        "emb_gamma": get("embeddings.LayerNorm.weight"),
        "emb_beta": get("embeddings.LayerNorm.bias"),
    }
    for l in range(layers):
        for i, name in enumerate(LAYER_ORDER):
            out[f"l{l}_{i:02d}"] = get(f"encoder.layer.{l}.{name}")
    return out


def main():
    eos = sys.argv[1]
    here = os.path.dirname(os.path.abspath(__file__))
    from safetensors.numpy import load_file

    fx = os.path.join(eos, "runtime/testdata/pretrained_bert_golden")
    cfg = json.load(open(os.path.join(fx, "config.json")))
    gold = json.load(open(os.path.join(fx, "golden.json")))
    state = load_file(os.path.join(fx, "model.safetensors"))
    arrays = pack_state(state, cfg["num_hidden_layers"])
    b = len(gold["texts"])
    t = gold["max_length"]
    arrays.update(
        input_ids=np.array(gold["input_ids"], dtype=np.int32).reshape(b, t),
        attention_mask=np.array(gold["attention_mask"], dtype=np.int32).reshape(b, t),
        token_type_ids=np.array(gold["token_type_ids"], dtype=np.int32).reshape(b, t),
        expected=np.array(gold["embeddings"], dtype=np.float32),
        layers=np.int32(cfg["num_hidden_layers"]), heads=np.int32(cfg["num_attention_heads"]),
        eps=np.float64(cfg["layer_norm_eps"]),
    )
    np.savez_compressed(os.path.join(here, "bert_tiny_golden.npz"), **arrays)

    import torch
    import torch.nn.functional as F
    from transformers import BertConfig, BertModel

    seed = 20261125
    config = BertConfig(vocab_size=50, hidden_size=64, num_hidden_layers=3, num_attention_heads=4,
                        intermediate_size=128, hidden_act="gelu", max_position_embeddings=24, type_vocab_size=2,
                        layer_norm_eps=1e-12, position_embedding_type="absolute")
    torch.manual_seed(seed)
    model = BertModel(config, add_pooling_layer=False).eval()
    gen = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for _, param in sorted(model.named_parameters()):
            param.copy_((torch.rand(param.shape, generator=gen) - 0.5) * 0.4)
    lengths = [24, 1, 7, 16, 11]
    ids = torch.randint(0, 50, (5, 24), generator=gen)
    mask = torch.zeros(5, 24, dtype=torch.long)
    for i, n in enumerate(lengths):
        mask[i, :n] = 1
    types = torch.zeros(5, 24, dtype=torch.long)
    types[:, 12:] = 1
    with torch.no_grad():
        hs = model(input_ids=ids, attention_mask=mask, token_type_ids=types).last_hidden_state
        m = mask.unsqueeze(-1).float()
        pooled = (hs * m).sum(1) / m.sum(1)
        emb = F.normalize(pooled, dim=-1)
        cls = F.normalize(hs[:, 0], dim=-1)
    arrays = pack_state({k: v.detach().numpy() for k, v in model.state_dict().items()}, 3)
    arrays.update(input_ids=ids.numpy().astype(np.int32), attention_mask=mask.numpy().astype(np.int32),
                  token_type_ids=types.numpy().astype(np.int32), expected=emb.numpy().astype(np.float32),
                  expected_cls=cls.numpy().astype(np.float32), layers=np.int32(3), heads=np.int32(4),
                  eps=np.float64(1e-12))
    np.savez_compressed(os.path.join(here, "bert_hf_seeded.npz"), **arrays)
    print("wrote fixtures to", here)


if __name__ == "__main__":
    main()
