"""Writes tests/golden/engine_hf.npz: logits of a tiny random Hugging Face Qwen2 (CPU, fp32, eager attention) whose
block linears hold codebook matrices decoded by the REFERENCE's decode_tensors - the pin of the decode engine.

    python tests/golden/make_engine_golden.py --ref /path/to/QuantExperiments

Needs `transformers` (CPU is enough).  The model is defined by seeds in tests/golden/tiny_qwen2.py, so the fixture
holds only the token ids and the logits [len(tokens), vocab] of every position."""
from __future__ import annotations

import argparse
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True, help="checkout of the reference repository")
    args = ap.parse_args()
    sys.path.insert(0, args.ref)
    import transformers
    from shapequant import packed as rp
    sys.path.insert(0, str(HERE))
    import tiny_qwen2 as tq

    cfg = transformers.Qwen2Config(hidden_size=tq.H, intermediate_size=tq.I, num_hidden_layers=tq.NL, num_attention_heads=tq.NH,
                                   num_key_value_heads=tq.NKV, vocab_size=tq.V, max_position_embeddings=tq.MAX_LEN,
                                   rope_parameters={"rope_type": "default", "rope_theta": tq.THETA}, rms_norm_eps=tq.EPS,
                                   tie_word_embeddings=False)
    cfg._attn_implementation = "eager"
    model = transformers.Qwen2ForCausalLM(cfg).float().eval()
    st = tq.small_tensors()
    names = {"q": "self_attn.q_proj", "k": "self_attn.k_proj", "v": "self_attn.v_proj", "o": "self_attn.o_proj",
             "gate": "mlp.gate_proj", "up": "mlp.up_proj", "down": "mlp.down_proj"}
    with torch.no_grad():
        sd = model.state_dict()
        sd["model.embed_tokens.weight"].copy_(torch.from_numpy(st["embed"]).float())
        sd["lm_head.weight"].copy_(torch.from_numpy(st["head"]).float())
        sd["model.norm.weight"].copy_(torch.from_numpy(st["final_norm"]).float())
        for li in range(tq.NL):
            sd[f"model.layers.{li}.input_layernorm.weight"].copy_(torch.from_numpy(st[f"ln1_{li}"]).float())
            sd[f"model.layers.{li}.post_attention_layernorm.weight"].copy_(torch.from_numpy(st[f"ln2_{li}"]).float())
            for n, hf in names.items():
                m = tq.matrix(li, n)
                tags = rp.unpack_bits(torch.from_numpy(m["words"][0]), 12, m["C"] // 8)
                w = rp.decode_tensors(tags, torch.from_numpy(m["table"][0]), torch.from_numpy(m["row_scale"]),
                                      torch.zeros(m["R"], dtype=torch.int64), None, torch.from_numpy(m["perms"]), 4096)
                sd[f"model.layers.{li}.{hf}.weight"].copy_(w)
                if n in "qkv":
                    sd[f"model.layers.{li}.{hf}.bias"].copy_(torch.from_numpy(st[f"b{n}_{li}"]).float())
        logits = model(torch.tensor([tq.TOKENS])).logits[0].float().numpy()
    np.savez_compressed(HERE / "engine_hf.npz", tokens=np.array(tq.TOKENS, np.int32), logits=logits)
    print("engine_hf.npz", logits.shape, float(np.abs(logits).max()))


if __name__ == "__main__":
    main()
