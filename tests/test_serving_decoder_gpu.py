"""GPU parity of the decoder harness (utils/decoder.py) on the config-2 model (4 layers, d_model 256, 4 heads, FFN
1024, vocab 65, context 128): the packed inference form against an eager copy with the same weights and against the
CPU oracle, projection by projection.  Structure under test: js/src/models/TernaryTransformer.ts:366-464, 520-600."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

VOCAB, DIM, LAYERS, HEADS, FFN, CTX, BATCH = 65, 256, 4, 4, 1024, 128, 8


def _models(backend_cuda="cuda", layers=LAYERS, fused_elementwise=True):
    """(eager model on the python backend, packed inference model) with identical weights, both on the GPU."""
    from bittorch_b200.utils.decoder import DecoderConfig, TernaryDecoder

    torch.manual_seed(0)
    cfg = dict(vocab_size=VOCAB, dim=DIM, n_layers=layers, n_heads=HEADS, ffn_dim=FFN, max_seq_len=CTX)
    eager = TernaryDecoder(DecoderConfig(backend="python", **cfg)).cuda().eval()
    packed = TernaryDecoder(DecoderConfig(backend=backend_cuda, fused_elementwise=fused_elementwise, **cfg)).cuda().eval()
    packed.load_state_dict(eager.state_dict())
    packed.to_inference()
    return eager, packed


def _teacher_forced_logits(model, tokens, prompt_len, fixed_shape):
    """Logits of every decode step when the model is fed `tokens` (prefill over the first prompt_len, then one token
    at a time against the cache)."""
    with torch.no_grad():
        cache = model.new_cache(tokens.shape[0])
        out = [model(tokens[:, :prompt_len], cache, 0)[:, -1]]
        for i in range(prompt_len, tokens.shape[1]):
            if fixed_shape:
                pos = torch.tensor([i], device=tokens.device)
                out.append(model.decode_step(tokens[:, i:i + 1], cache, pos)[:, -1])
            else:
                out.append(model(tokens[:, i:i + 1], cache, i)[:, -1])
    return torch.stack(out, dim=1)                             # [B, steps, vocab]


def _agree_where_clear(a, b, margin):
    """arg-max of a and b agree wherever a's best logit leads its runner-up by more than `margin`."""
    top = a.topk(2, dim=-1).values
    clear = (top[..., 0] - top[..., 1]) > margin
    return bool((a.argmax(-1) == b.argmax(-1))[clear].all()), float(clear.float().mean())


def test_float_mode_matches_the_eager_model(monkeypatch):
    """BITTORCH_B200_ACT=float (the reference's fp32-accumulate arithmetic): 128 greedy tokens of the eager model, fed
    to both models; logits agree within 1e-4 (relative to their scale) at every step and the greedy choice is the
    same wherever it is not a numerical tie."""
    monkeypatch.setenv("BITTORCH_B200_ACT", "float")
    eager, packed = _models()
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, VOCAB, (BATCH, 1), generator=g).cuda()
    tokens = eager.generate_greedy(prompt, CTX - 1)            # positions 0 .. 127
    la = _teacher_forced_logits(eager, tokens, 1, fixed_shape=False)
    lb = _teacher_forced_logits(packed, tokens, 1, fixed_shape=False)
    scale = float(la.abs().max())
    assert float((la - lb).abs().max()) <= 1e-4 * max(scale, 1.0) + 1e-4
    same, clear = _agree_where_clear(la, lb, 1e-3 * max(scale, 1.0))
    assert same and clear > 0.9
    lc = _teacher_forced_logits(packed, tokens, 1, fixed_shape=True)      # the graph-friendly step, same arithmetic
    assert float((la - lc).abs().max()) <= 1e-4 * max(scale, 1.0) + 1e-4


def test_every_projection_is_the_oracles_integer_chain(oracle):
    """Integer mode: hooks capture the input and output of every packed projection during a prefill ([8, 5] tokens ->
    40 rows, tensor-core kernel) and a decode step of 2 sequences (decode kernel); each output must equal the
    oracle's quantize -> integer contraction -> epilogue on the captured input, bit for bit.  The fused q/kv and
    gate/up launches are covered through their members' columns."""
    from bittorch_b200.nn import TernaryLinearInference
    from bittorch_b200.utils.decoder import fuse_inference_columns

    _, packed = _models(layers=2, fused_elementwise=False)     # module by module: the forward hooks see every projection
    calls = []
    hooks = []

    def watch(name, mod):
        hooks.append(mod.register_forward_hook(lambda m, inp, out: calls.append((name, m, inp[0].detach(), out.detach()))))

    for name, mod in packed.named_modules():
        if isinstance(mod, TernaryLinearInference):
            watch(name, mod)
    # fused siblings are private modules (not in named_modules): watch them through their owners after the first call
    g = torch.Generator().manual_seed(2)
    tokens = torch.randint(0, VOCAB, (BATCH, 5), generator=g).cuda()
    with torch.no_grad():
        cache = packed.new_cache(BATCH)
        packed(tokens, cache, 0)
        for blk in packed.blocks:
            watch("fused_qkv", blk.attn._fused._fused)
            watch("fused_gate_up", blk.mlp._fused._fused)
        calls.clear()
        packed(tokens, cache, 0)                               # 40 rows per projection
        cache2 = packed.new_cache(2)
        packed(tokens[:2, :1], cache2, 0)                      # 2 rows per projection
    for h in hooks:
        h.remove()
    assert len(calls) == 2 * 2 * 4                             # 2 passes x 2 blocks x (fused qkv, proj, fused gate/up, down)
    seen_rows = set()
    for name, mod, x, y in calls:
        k, n = mod.in_features, mod.out_features
        codes = oracle.unpack_transposed(mod.public_packed().cpu().numpy(), k)
        x2 = x.reshape(-1, k).float().cpu().numpy()
        q, sx = oracle.act_quant(x2)
        y_ref = oracle.epilogue(oracle.gemm_i32(q, codes), sx, mod.scale.float().cpu().numpy(), None)
        assert np.array_equal(y.reshape(-1, n).cpu().numpy().view(np.uint32), y_ref.view(np.uint32)), name
        seen_rows.add(x2.shape[0])
    assert seen_rows == {40, 2}

    # one fused launch == its members, bit for bit
    blk = packed.blocks[0]
    x = torch.randn(3, DIM, generator=g).cuda()
    with torch.no_grad():
        fused = fuse_inference_columns([blk.attn.q_proj, blk.attn.kv_proj])(x)
        assert torch.equal(fused, torch.cat([blk.attn.q_proj(x), blk.attn.kv_proj(x)], dim=-1))
        fused = fuse_inference_columns([blk.mlp.w_gate, blk.mlp.w_up])(x)
        assert torch.equal(fused, torch.cat([blk.mlp.w_gate(x), blk.mlp.w_up(x)], dim=-1))


def test_integer_mode_tracks_the_eager_model():
    """Integer mode against the eager float model: not gated at 1e-3 (per-token int8 activations deviate by about
    1e-2 of the output norm per layer), reported through a loose bound on the logits of a 4-layer model."""
    eager, packed = _models()
    g = torch.Generator().manual_seed(3)
    tokens = torch.randint(0, VOCAB, (BATCH, 16), generator=g).cuda()
    with torch.no_grad():
        la, lb = eager(tokens), packed(tokens)
    rel = float((la - lb).norm() / la.norm())
    assert rel < 0.15, rel


def test_graph_replayed_greedy_loop_equals_the_eager_steps():
    """GreedyDecodeGraph (one CUDA-graph launch per token: decode step, arg-max, position counter on the device)
    produces exactly the tokens of the same steps run eagerly, and keeps the cache identical."""
    from bittorch_b200.utils.decoder import GreedyDecodeGraph

    _, packed = _models()
    g = torch.Generator().manual_seed(4)
    prompt = torch.randint(0, VOCAB, (BATCH, 6), generator=g).cuda()
    steps = 40
    with torch.no_grad():
        cache_a = packed.new_cache(BATCH)
        first = packed(prompt, cache_a, 0)[:, -1].argmax(dim=-1, keepdim=True)
        cache_b = [(k.clone(), v.clone()) for k, v in cache_a]
        # eager: the same fixed-shape step, driven from the host
        want, tok = [], first
        for i in range(steps):
            want.append(tok)
            logits = packed.decode_step(tok, cache_a, torch.tensor([6 + i], device=tok.device))
            tok = logits[:, -1].argmax(dim=-1, keepdim=True)
        want = torch.cat(want, dim=1)
    loop = GreedyDecodeGraph(packed, BATCH, cache=cache_b)
    loop.start(first, 6)
    loop.run(steps)
    torch.cuda.synchronize()
    assert torch.equal(loop.history[:, 6:6 + steps], want)
    assert torch.equal(loop.tokens, tok)
    for (ka, va), (kb, vb) in zip(cache_a, cache_b):
        assert torch.equal(ka, kb) and torch.equal(va, vb)
    # a second generation from the same graph
    loop.start(first, 6)
    loop.run(steps)
    torch.cuda.synchronize()
    assert torch.equal(loop.history[:, 6:6 + steps], want)


def test_inference_form_keeps_one_copy_of_the_weights_and_checkpoints_do_not_change(tmp_path):
    """to_inference() with one_weight_copy (the default): after the first forward every projection holds only the
    tiled copy (the fused pairs share one buffer with their members), so device bytes per projection are
    ceil(K/4) * N; the state dict still carries the public `weight_packed` buffers, byte for byte what a model
    without the option holds; loading it into a fresh model reproduces the logits."""
    from bittorch_b200.nn import TernaryLinearInference
    from bittorch_b200.utils.decoder import DecoderConfig, TernaryDecoder

    torch.manual_seed(5)
    cfg = dict(vocab_size=VOCAB, dim=DIM, n_layers=2, n_heads=HEADS, ffn_dim=FFN, max_seq_len=32)
    masters = TernaryDecoder(DecoderConfig(backend="python", **cfg)).cuda().eval()
    two = TernaryDecoder(DecoderConfig(backend="cuda", one_weight_copy=False, **cfg)).cuda().eval()
    one = TernaryDecoder(DecoderConfig(backend="cuda", **cfg)).cuda().eval()
    for m in (two, one):
        m.load_state_dict(masters.state_dict())
        m.to_inference()
    tokens = torch.randint(0, VOCAB, (3, 7), generator=torch.Generator().manual_seed(6)).cuda()
    with torch.no_grad():
        want = two(tokens)
        got = one(tokens)
        got_again = one(tokens)
    assert torch.equal(got, want) and torch.equal(got_again, want)

    weight_bytes = 0
    storages = set()
    for name, mod in one.named_modules():
        if isinstance(mod, TernaryLinearInference):
            assert mod._compact and mod.weight_packed.numel() == 0, name
            assert mod._tiled.numel() == mod.packed_size_bytes            # dims are multiples of the tile: no padding
            storages.add(mod._tiled.untyped_storage().data_ptr())
            weight_bytes += mod._tiled.numel()
    per_block = (DIM * DIM + DIM * 2 * DIM + DIM * DIM + 3 * DIM * FFN) // 4
    assert weight_bytes == 2 * per_block
    assert len(storages) == 2 * 4                                          # per block: fused q/kv, proj, fused gate/up, down
    for blk in one.blocks:                                                 # the fused layers own what the members view
        assert blk.attn._fused._fused._tiled.untyped_storage().data_ptr() == blk.attn.q_proj._tiled.untyped_storage().data_ptr()
        assert blk.mlp._fused._fused._tiled.untyped_storage().data_ptr() == blk.mlp.w_up._tiled.untyped_storage().data_ptr()

    sd_one, sd_two = one.state_dict(), two.state_dict()
    assert set(sd_one) == set(sd_two)
    for key in sd_two:
        assert torch.equal(sd_one[key], sd_two[key]), key                  # wire format unchanged, byte for byte
    path = str(tmp_path / "decoder.pt")
    torch.save(sd_one, path)
    fresh = TernaryDecoder(DecoderConfig(backend="cuda", **cfg)).cuda().eval()
    fresh.load_state_dict(masters.state_dict())
    fresh.to_inference()
    fresh.load_state_dict(torch.load(path))
    with torch.no_grad():
        assert torch.equal(fresh(tokens), want)


def test_fused_elementwise_blocks_follow_the_unfused_model():
    """The inference form with residual add + RMSNorm and SiLU * up inside the quantizer kernels
    (bt_add_rmsnorm_quant, bt_silu_mul_quant; the kernels themselves are pinned bit for bit elsewhere) against the
    same model with those steps as framework operations: the two differ only where the framework's own summation
    order or exponential rounds a value the other way, so logits agree closely, over a prefill, a growing-shape
    step and a fixed-shape step; fp32 and bf16 models."""
    from bittorch_b200.utils.decoder import DecoderConfig, TernaryDecoder

    for dtype, tol in ((torch.float32, 2e-3), (torch.bfloat16, 6e-2)):
        torch.manual_seed(7)
        cfg = dict(vocab_size=VOCAB, dim=DIM, n_layers=2, n_heads=HEADS, n_kv_heads=2, ffn_dim=FFN, max_seq_len=32)
        masters = TernaryDecoder(DecoderConfig(backend="python", **cfg)).cuda().eval()
        models = []
        for fused in (False, True):
            m = TernaryDecoder(DecoderConfig(backend="cuda", fused_elementwise=fused, **cfg)).cuda().eval()
            m.load_state_dict(masters.state_dict())
            models.append(m.to(dtype).to_inference())
        plain, fused = models
        assert fused._fused_blocks() and not plain._fused_blocks()
        tokens = torch.randint(0, VOCAB, (3, 9), generator=torch.Generator().manual_seed(8)).cuda()
        with torch.no_grad():
            ca, cb = plain.new_cache(3), fused.new_cache(3)
            pairs = [(plain(tokens[:, :7], ca, 0), fused(tokens[:, :7], cb, 0)),
                     (plain(tokens[:, 7:8], ca, 7), fused(tokens[:, 7:8], cb, 7)),
                     (plain.decode_step(tokens[:, 8:9], ca, torch.tensor([8], device=tokens.device)),
                      fused.decode_step(tokens[:, 8:9], cb, torch.tensor([8], device=tokens.device)))]
            # a prefill that asks for the last position only gets the same logits for it (the head's matrix product
            # over one row instead of seven may round its sums in another order)
            for m, full in ((plain, pairs[0][0]), (fused, pairs[0][1])):
                last = m(tokens[:, :7], m.new_cache(3), 0, last_only=True)
                assert last.shape == full[:, -1:].shape
                assert float((last.float() - full[:, -1:].float()).norm() / full[:, -1:].float().norm()) < tol / 10
        for a, b in pairs:
            assert a.shape == b.shape
            rel = float((a.float() - b.float()).norm() / a.float().norm())
            assert rel < tol, (dtype, rel)
