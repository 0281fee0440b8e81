"""The plain implementation: against the reference's own model code (the committed golden
numbers of tests/golden/), and each of its parts against a direct evaluation of its formula."""
import math
import os

import torch
from safetensors.torch import load_file

import plain_qwen3 as plain

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _golden():
    cfg, w = plain.read_model_folder(os.path.join(GOLDEN, "model"))
    return cfg, w, load_file(os.path.join(GOLDEN, "golden.safetensors"))


def test_whole_prompt_equals_reference_prefill():
    cfg, w, g = _golden()
    got = plain.forward_logits(cfg, w, g["whole.tokens"].tolist())
    assert float((got - g["whole.logits"]).abs().max()) < 2e-5


def test_decode_steps_equal_reference_decode():
    cfg, w, g = _golden()
    toks = g["whole.tokens"].tolist() + g["decode.tokens"].tolist()
    got = plain.forward_logits(cfg, w, toks)[-4:]
    assert float((got - g["decode.logits"]).abs().max()) < 2e-5


def test_shared_prefix_rows_equal_reference():
    cfg, w, g = _golden()
    got = plain.forward_logits(cfg, w, g["shared.tokens"].tolist())[16:]
    assert float((got - g["shared.logits"]).abs().max()) < 2e-5


def test_rmsnorm_formula():
    x = torch.tensor([[3.0, -4.0, 0.0, 12.0]])
    w = torch.tensor([1.0, 2.0, 3.0, 0.5])
    eps = 1e-3
    rms = math.sqrt((9 + 16 + 0 + 144) / 4 + eps)
    want = torch.tensor([[3 / rms, -8 / rms, 0.0, 6 / rms]])
    assert torch.allclose(plain.rmsnorm(x, w, eps), want, atol=1e-6)


def test_rope_is_a_rotation_of_half_split_pairs():
    D, theta = 8, 100.0
    x = torch.arange(1, D + 1, dtype=torch.float32).view(1, 1, D)
    pos = torch.tensor([3])
    cos, sin = plain.rope_angles(pos, D, theta)
    y = plain.rope_rotate(x, cos, sin)[0, 0]
    for j in range(D // 2):
        ang = 3 * theta ** (-2 * j / D)
        a, b = float(x[0, 0, j]), float(x[0, 0, j + D // 2])
        assert abs(float(y[j]) - (math.cos(ang) * a - math.sin(ang) * b)) < 1e-5
        assert abs(float(y[j + D // 2]) - (math.sin(ang) * a + math.cos(ang) * b)) < 1e-5
    # position 0 leaves the vector alone; norms are kept
    cos0, sin0 = plain.rope_angles(torch.tensor([0]), D, theta)
    assert torch.equal(plain.rope_rotate(x, cos0, sin0), x)
    assert abs(float(y.norm()) - float(x.norm())) < 1e-4


def test_attention_is_causal_and_grouped():
    torch.manual_seed(0)
    T, Hq, Hkv, D = 6, 4, 2, 8
    q, k, v = torch.randn(T, Hq, D), torch.randn(T, Hkv, D), torch.randn(T, Hkv, D)
    out = plain.causal_attention(q, k, v, 0.3)
    # the first query sees only the first key: its output is v[0] of its group
    for h in range(Hq):
        assert torch.allclose(out[0, h], v[0, h // 2], atol=1e-6)
    # changing a later key or value does not change an earlier output
    k2, v2 = k.clone(), v.clone()
    k2[4:] += 5.0
    v2[4:] -= 3.0
    out2 = plain.causal_attention(q, k2, v2, 0.3)
    assert torch.equal(out[:4], out2[:4])
    # explicit softmax for one (query, head)
    s = torch.stack([(q[3, 2] * k[j, 1]).sum() * 0.3 for j in range(4)])
    p = torch.softmax(s, 0)
    assert torch.allclose(out[3, 2], (p[:, None] * v[:4, 1]).sum(0), atol=1e-6)
    # a window of 2 keeps keys i-1 and i
    outw = plain.causal_attention(q, k, v, 0.3, window=2)
    s = torch.stack([(q[3, 0] * k[j, 0]).sum() * 0.3 for j in (2, 3)])
    p = torch.softmax(s, 0)
    assert torch.allclose(outw[3, 0], p[0] * v[2, 0] + p[1] * v[3, 0], atol=1e-6)


def test_silu_mul_formula():
    g = torch.tensor([0.0, 1.0, -2.0])
    u = torch.tensor([5.0, 2.0, 3.0])
    want = torch.tensor([0.0, 2.0 / (1 + math.exp(-1.0)), -6.0 / (1 + math.exp(2.0))])
    assert torch.allclose(plain.silu_mul(g, u), want, atol=1e-6)


def test_tied_head_uses_the_embedding(model_folders):
    cfg, w = plain.read_model_folder(model_folders["tiny-a"])
    assert cfg["tie_word_embeddings"] and "lm_head.weight" not in w
    logits = plain.forward_logits(cfg, w, [1, 2, 3])
    assert logits.shape == (3, cfg["vocab_size"])


def test_greedy_generate_is_repeated_argmax(model_folders):
    cfg, w = plain.read_model_folder(model_folders["tiny-b"])
    prompt = [5, 17, 3, 200]
    out = plain.greedy_generate(cfg, w, prompt, 3)
    assert out[0] == int(plain.forward_logits(cfg, w, prompt)[-1].argmax())
    assert out[1] == int(plain.forward_logits(cfg, w, prompt + out[:1])[-1].argmax())


def test_the_smoke_tests_model_with_head_size_128_has_clear_first_choices(tmp_path):
    """`__graft_entry__.smoke()` compares bfloat16 tokens with the plain implementation only while the plain choice is
    clear (the best logit leads by more than 6 % of the largest); its model with head size 128 must give it something
    to compare: at least three of its four tokens."""
    import os
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import __graft_entry__ as entry
    from qwen_engine_b200.weights import write_model_folder
    cfg, init, prompt = entry.smoke_model_d128()
    folder = write_model_folder(cfg, str(tmp_path / "d128"), *init)
    pc, pw = plain.read_model_folder(folder)
    want = plain.greedy_generate(pc, pw, prompt, 4)
    assert entry._same_tokens_while_clear(plain, pc, pw, prompt, want, want, "plain against itself") >= 3
