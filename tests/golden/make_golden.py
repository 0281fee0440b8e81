"""Makes tests/golden/: logits of kzw3933/Qwen-Engine's own model code for a tiny random model.

Run once on a machine where the reference's sources can be imported (CPU is enough; its
``mode="torch"`` path is plain PyTorch):

    python tests/golden/make_golden.py /path/to/Qwen-Engine

It writes, next to itself,
  model/config.json, model/model.safetensors   a tiny float32 Qwen3 model (seeded here, 25 k weights)
  golden.safetensors                            token ids and the reference's logits:
      whole.tokens / whole.logits        a 23-token prompt through run_prefill (all rows)
      decode.logits                      4 more tokens one by one through run_decode_step
      shared.tokens / shared.logits      a prompt sharing 16 tokens with the first: the rows the
                                         reference computes after taking the shared pages

tests/test_plain.py compares tests/plain_qwen3.py with these numbers; nothing here is imported by
the engine.
"""
import json
import os
import sys

import torch
from safetensors.torch import save_file

HERE = os.path.dirname(os.path.abspath(__file__))

CONFIG = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=32, num_attention_heads=4,
              num_key_value_heads=2, head_dim=16, intermediate_size=48, vocab_size=61, rope_theta=10000.0,
              rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=128, attention_bias=False,
              hidden_act="silu")


def main(ref_root: str) -> None:
    sys.dont_write_bytecode = True
    sys.path.insert(0, os.path.join(ref_root, "src"))
    from models import Qwen3Config, Qwen3ForCausalLM          # the reference's own classes
    from engine import KVCachePool
    from engine.executor import ModelExecutor
    from engine.sequence import Sequence

    torch.manual_seed(1234)
    cfg = Qwen3Config(head_dim=16, hidden_size=32, intermediate_size=48, max_position_embeddings=128,
                      num_attention_heads=4, num_hidden_layers=2, num_key_value_heads=2, rms_norm_eps=1e-5,
                      rope_theta=10000, tie_word_embeddings=False, vocab_size=61)
    model = Qwen3ForCausalLM(**cfg.to_model_kwargs(), dtype=torch.float32).eval()
    with torch.no_grad():
        for name, p in model.named_parameters():
            if name.endswith("norm.weight") or "layernorm" in name:
                p.copy_(1.0 + 0.2 * torch.randn_like(p))
            else:
                p.copy_(0.08 * torch.randn_like(p))
    os.makedirs(os.path.join(HERE, "model"), exist_ok=True)
    with open(os.path.join(HERE, "model", "config.json"), "w") as f:
        json.dump(CONFIG, f, indent=2, sort_keys=True)
        f.write("\n")
    save_file({n: p.detach().clone().contiguous() for n, p in model.named_parameters()},
              os.path.join(HERE, "model", "model.safetensors"), metadata={"format": "pt"})

    g = torch.Generator().manual_seed(99)
    whole = torch.randint(0, 61, (23,), generator=g).tolist()
    more = torch.randint(0, 61, (4,), generator=g).tolist()
    shared = whole[:16] + torch.randint(0, 61, (9,), generator=g).tolist()
    pool = KVCachePool(num_layers=2, num_blocks=16, block_size=8, num_kv_heads=2, head_dim=16,
                       dtype=torch.float32, device=torch.device("cpu"))
    ex = ModelExecutor(model, pool, torch.device("cpu"), mode="torch")
    out = {}
    with torch.no_grad():
        s1 = Sequence(0, "", list(whole))
        logits, _ = ex.run_prefill([s1])
        out["whole.tokens"] = torch.tensor(whole, dtype=torch.int32)
        out["whole.logits"] = logits.clone()
        s2 = Sequence(1, "", list(shared))
        logits2, ctx2 = ex.run_prefill([s2])
        assert s2.shared_prefix_len == 16
        out["shared.tokens"] = torch.tensor(shared, dtype=torch.int32)
        out["shared.logits"] = logits2.clone()                 # rows 16 .. 24 of the prompt
        s1.num_computed_tokens = s1.num_kv_tokens = s1.prompt_len
        rows = []
        for t in more:                                         # teacher-forced decode steps
            s1.output_token_ids.append(t)
            rows.append(ex.run_decode_step([s1])[0].clone())
            s1.num_computed_tokens += 1
            s1.num_kv_tokens += 1
        out["decode.tokens"] = torch.tensor(more, dtype=torch.int32)
        out["decode.logits"] = torch.stack(rows)
    save_file(out, os.path.join(HERE, "golden.safetensors"))
    print({k: tuple(v.shape) for k, v in out.items()})


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/Qwen-Engine")
    main(sys.argv[1])
