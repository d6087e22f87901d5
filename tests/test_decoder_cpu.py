"""CPU checks of the decoder that drives the ternary layers the way a language model does
(python backend of the layers, so no GPU): its pieces against direct restatements of the browser
runtime's loops (js/src/core/RMSNorm.ts, js/src/core/RoPE.ts, js/src/models/TernaryTransformer.ts),
and decoding against a key/value cache against recomputing the whole sequence."""

import math

import numpy as np
import pytest
import torch

from bittorch_b200.utils.decoder import (DecoderConfig, RMSNorm, TernaryDecoder, apply_rope, rope_tables)


def _cfg(**kw):
    base = dict(vocab_size=65, dim=64, n_layers=2, n_heads=4, n_kv_heads=2, ffn_dim=96, max_seq_len=24, backend="python")
    base.update(kw)
    return DecoderConfig(**base)


def test_rmsnorm_is_the_runtimes_loop():
    torch.manual_seed(0)
    x = torch.randn(3, 16)
    m = RMSNorm(16)
    with torch.no_grad():
        m.weight.copy_(torch.randn(16))
    y = m(x).detach().numpy()
    xn, w = x.numpy().astype(np.float64), m.weight.detach().numpy().astype(np.float64)
    for t in range(3):
        rms = math.sqrt((xn[t] ** 2).sum() / 16 + 1e-5)
        assert np.allclose(y[t], xn[t] / rms * w, atol=1e-6)


def test_rope_pairs_element_i_with_i_plus_half():
    head_dim, seq = 8, 5
    cos, sin = rope_tables(16, head_dim)
    x = torch.randn(1, 2, seq, head_dim, dtype=torch.float64)
    y = apply_rope(x, cos.double(), sin.double(), pos0=3).numpy()
    xn = x.numpy()
    half = head_dim // 2
    for h in range(2):
        for t in range(seq):
            for i in range(half):
                angle = (3 + t) * (1.0 / 10000.0 ** (2 * i / head_dim))
                x0, x1 = xn[0, h, t, i], xn[0, h, t, i + half]
                assert abs(y[0, h, t, i] - (x0 * math.cos(angle) - x1 * math.sin(angle))) < 1e-6
                assert abs(y[0, h, t, i + half] - (x0 * math.sin(angle) + x1 * math.cos(angle))) < 1e-6


def test_parameter_names_are_the_runtimes_checkpoint_names():
    names = set(dict(TernaryDecoder(_cfg()).named_parameters()))
    want = {"tok.weight", "norm.weight", "head.weight"}
    for i in range(2):
        want |= {f"blocks.{i}.norm1.weight", f"blocks.{i}.norm2.weight"}
        want |= {f"blocks.{i}.attn.{p}.weight" for p in ("q_proj", "kv_proj", "proj")}
        want |= {f"blocks.{i}.mlp.{p}.weight" for p in ("w_gate", "w_up", "w_down")}
    assert names == want


@pytest.mark.parametrize("n_kv_heads", [4, 2, 1])
def test_decoding_against_the_cache_equals_recomputing_the_sequence(n_kv_heads):
    torch.manual_seed(1)
    model = TernaryDecoder(_cfg(n_kv_heads=n_kv_heads)).eval()
    tokens = torch.randint(0, 65, (2, 10))
    with torch.no_grad():
        full = model(tokens)                                   # one pass over all ten positions
        cache = model.new_cache(2)
        pre = model(tokens[:, :6], cache, 0)                   # prefill six, then four single-token steps
        steps = [model(tokens[:, 6 + i:7 + i], cache, 6 + i) for i in range(4)]
        last = model(tokens[:, :6], model.new_cache(2), 0, last_only=True)
    assert torch.allclose(pre, full[:, :6], atol=1e-5)
    assert last.shape == (2, 1, 65) and torch.allclose(last, pre[:, -1:], atol=1e-5)     # a prefill's logits: the last position alone
    for i, s in enumerate(steps):
        assert torch.allclose(s[:, 0], full[:, 6 + i], atol=1e-5)


def test_attention_is_the_runtimes_loop_for_one_head_group():
    """One block's attention output against the runtime's scalar loops (scores over keys 0..tq, softmax, weighted
    sum of values; query head h reads key/value head h // group), with the projections as plain matrices."""
    torch.manual_seed(2)
    cfg = _cfg(n_layers=1, dim=16, n_heads=4, n_kv_heads=2, ffn_dim=16)
    model = TernaryDecoder(cfg).eval()
    attn = model.blocks[0].attn
    x = torch.randn(1, 5, 16)
    with torch.no_grad():
        cache = model.new_cache(1)[0]
        got = attn(x, cache, 0, model.rope_cos, model.rope_sin)
        q = attn.q_proj(x)[0].numpy().astype(np.float64)           # [T, dim]
        kv = attn.kv_proj(x)[0].numpy().astype(np.float64)         # [T, 2 * kv_dim]
    hd, nh, nkv, seq = 4, 4, 2, 5
    kv_dim = nkv * hd
    cos, sin = rope_tables(cfg.max_seq_len, hd)
    cos, sin = cos.numpy().astype(np.float64), sin.numpy().astype(np.float64)

    def rope(vec, pos):
        out = vec.copy()
        for i in range(hd // 2):
            out[i] = vec[i] * cos[pos, i] - vec[i + hd // 2] * sin[pos, i]
            out[i + hd // 2] = vec[i] * sin[pos, i] + vec[i + hd // 2] * cos[pos, i]
        return out

    out = np.zeros((seq, 16))
    for h in range(nh):
        kh = h // (nh // nkv)
        for tq in range(seq):
            qv = rope(q[tq, h * hd:(h + 1) * hd], tq)
            scores = np.array([qv @ rope(kv[tk, kh * hd:(kh + 1) * hd], tk) / math.sqrt(hd) for tk in range(tq + 1)])
            p = np.exp(scores - scores.max())
            p /= p.sum()
            out[tq, h * hd:(h + 1) * hd] = sum(p[tk] * kv[tk, kv_dim + kh * hd:kv_dim + (kh + 1) * hd] for tk in range(tq + 1))
    with torch.no_grad():
        want = attn.proj(torch.from_numpy(out).float()[None])
    assert torch.allclose(got, want, atol=1e-5)


def test_greedy_generation_extends_the_prompt_and_respects_the_context_limit():
    torch.manual_seed(3)
    model = TernaryDecoder(_cfg()).eval()
    prompt = torch.randint(0, 65, (3, 4))
    out = model.generate_greedy(prompt, 6)
    assert out.shape == (3, 10) and torch.equal(out[:, :4], prompt)
    # the same tokens come out of recomputing the whole sequence at every step
    seq = prompt
    with torch.no_grad():
        for _ in range(6):
            seq = torch.cat([seq, model(seq)[:, -1].argmax(dim=-1, keepdim=True)], dim=1)
    assert torch.equal(out, seq)
    with pytest.raises(ValueError, match="max_seq_len"):
        model(torch.zeros(1, 25, dtype=torch.long))


def test_fused_sibling_layers_are_the_members_columns_side_by_side(oracle):
    """Gate/up (and q/kv) run as one packed layer in the inference form: its buffers are the members' buffers
    concatenated along the output columns, i.e. exactly the packed form of the concatenated weights."""
    from bittorch_b200.nn import TernaryLinearInference
    from bittorch_b200.utils.decoder import fuse_inference_columns

    rng = np.random.default_rng(0)
    k = 37                                                   # ragged K: 10 packed bytes per column
    codes = [rng.integers(-1, 2, size=(n, k)).astype(np.int8) for n in (24, 9)]
    scales = [rng.random(n).astype(np.float32) + 0.1 for n in (24, 9)]
    layers = [TernaryLinearInference(k, c.shape[0], torch.from_numpy(oracle.pack_transposed(c)), torch.from_numpy(s),
                                     torch.from_numpy(s * 2) if i == 1 else None)
              for i, (c, s) in enumerate(zip(codes, scales))]
    fused = fuse_inference_columns(layers)
    assert fused.in_features == k and fused.out_features == 33
    assert np.array_equal(fused.weight_packed.numpy(), oracle.pack_transposed(np.concatenate(codes, axis=0)))
    assert np.array_equal(fused.scale.numpy(), np.concatenate(scales))
    assert np.array_equal(fused.bias.numpy(), np.concatenate([np.zeros(24, np.float32), scales[1] * 2]))
    with pytest.raises(ValueError, match="same input"):
        fuse_inference_columns([layers[0], TernaryLinearInference(k + 4, 9, layers[1].weight_packed, layers[1].scale)])


@pytest.mark.parametrize("n_kv_heads", [4, 2, 1])
def test_fixed_shape_decode_step_equals_the_growing_shape_step(n_kv_heads):
    """decode_step (position in a tensor, attention over the whole cache under a mask) against forward (position as
    an integer, attention over the filled part): same logits and same cache contents (to float tolerance: the attention arithmetic differs), step after step."""
    torch.manual_seed(3)
    model = TernaryDecoder(_cfg(n_kv_heads=n_kv_heads)).eval()
    tokens = torch.randint(0, 65, (2, 9))
    with torch.no_grad():
        cache_a, cache_b = model.new_cache(2), model.new_cache(2)
        model(tokens[:, :5], cache_a, 0)
        model(tokens[:, :5], cache_b, 0)
        for i in range(5, 9):
            want = model(tokens[:, i:i + 1], cache_a, i)
            got = model.decode_step(tokens[:, i:i + 1], cache_b, torch.tensor([i]))
            assert torch.allclose(got, want, atol=1e-5)
        for (ka, va), (kb, vb) in zip(cache_a, cache_b):
            assert torch.allclose(ka, kb, atol=1e-5) and torch.allclose(va, vb, atol=1e-5)   # two softmax codes upstream


def test_greedy_decode_graph_produces_generate_greedys_tokens():
    """GreedyDecodeGraph with the capture replaced by a plain callable (no GPU here): the device-side loop (token
    buffer, position counter, history) yields the tokens of generate_greedy."""
    from bittorch_b200.utils.decoder import GreedyDecodeGraph

    class Replayable:
        def __init__(self, fn):
            self.fn = fn

        def replay(self):
            self.fn()

    def capture(step_fn, reset):
        for _ in range(3):                                    # like the real capture: warm-up calls, each undone
            step_fn()
            reset()
        return Replayable(step_fn)

    torch.manual_seed(4)
    model = TernaryDecoder(_cfg()).eval()
    prompt = torch.randint(0, 65, (3, 4))
    want = model.generate_greedy(prompt, 8)
    with torch.no_grad():
        cache = model.new_cache(3)
        first = model(prompt, cache, 0)[:, -1].argmax(dim=-1, keepdim=True)
    loop = GreedyDecodeGraph(model, 3, cache=cache, capture=capture)
    loop.start(first, 4)
    loop.run(8)
    assert torch.equal(loop.history[:, 4:12], want[:, 4:12])
    with pytest.raises(ValueError):
        loop.run(24)
