"""The minimal DRT body: host-side pieces on CPU, and on the GPU the reference's one behavioural
pin of the decode path -- greedy incremental decoding reproduces the argmax of a teacher-forced
forward over the generated sequence (``tests/generation_unittest.py:16-37``: tiny DRT with two
retrieval groups, 126 prompt tokens, 126 generated)."""
import math

import pytest
import torch

from long_context_modeling_b200 import drt_minimal as D


def tiny_config():
    return D.DRTConfig(hidden_size=128, num_attention_heads=2, intermediate_size=512, vocab_size=100,
                       decoder_layers=[1, 1, 1], encoder_layers=1, enc_chunk_size=63, chunk_topk=8,
                       slide_window=512, chunk_id=99)


@pytest.mark.parametrize("l,window", [(50, 16), (128, 32), (200, 64), (64, 512)])
def test_windowed_alibi_attention_matches_dense_mask(l, window):
    g = torch.Generator().manual_seed(l)
    n, h, d = 2, 3, 16
    q, k, v = (torch.randn(n, h, l, d, generator=g) for _ in range(3))
    slopes = D.alibi_slopes(h)
    got = D.windowed_alibi_attention(q, k, v, window, slopes)
    i = torch.arange(l).view(l, 1)
    j = torch.arange(l).view(1, l)
    dist = (i - j).float()
    bias = (-slopes.view(h, 1, 1) * dist).masked_fill((dist < 0) | (dist > window), float("-inf"))
    ref = torch.softmax(q @ k.transpose(-1, -2) / math.sqrt(d) + bias, -1) @ v
    assert (got - ref).abs().max().item() < 1e-5


def test_landmark_insertion_and_loss_targets():
    m = D.DRTMinimal(tiny_config())
    tok = torch.arange(126).view(1, 126) % 90
    ids = m.insert_landmarks(tok)
    assert ids.shape == (1, 128)
    assert ids[0, 63].item() == 99 and ids[0, 127].item() == 99
    assert torch.equal(ids[0, :63], tok[0, :63]) and torch.equal(ids[0, 64:127], tok[0, 63:])
    with pytest.raises(ValueError):
        m.insert_landmarks(tok[:, :100])


@pytest.mark.gpu
def test_incremental_decoding_equals_teacher_forced_argmax():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    torch.manual_seed(0)
    model = D.DRTMinimal(tiny_config()).cuda().eval()
    prompt = torch.randint(0, 99, (1, 126), device="cuda")
    out = model.generate(prompt, 126)
    assert out.shape == (1, 252)
    with torch.no_grad():
        logits = model(out)
    pred = logits.argmax(-1)
    assert torch.equal(pred[0, 125:-1], out[0, 126:])


@pytest.mark.gpu
@pytest.mark.parametrize("segment_chunks", [1, 2, 3])
def test_segmented_prefill_equals_monolithic(segment_chunks):
    """A long prompt prefilled segment by segment (self-attention window and chunk cache carried over,
    ``model/DRT.py:1018-1050``) gives the logits, the retrieved chunks and the next decoded tokens of the
    one-pass prefill."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    torch.manual_seed(3)
    cfg = tiny_config()
    cfg.slide_window = 40                                      # shorter than a chunk: the window crosses segments
    model = D.DRTMinimal(cfg).cuda().eval()
    prompt = torch.randint(0, 99, (2, 63 * 6), device="cuda")
    with torch.no_grad():
        s_mono = D.DecodeState(cfg)
        mono = model(prompt, state=s_mono)
        seg, s_seg = model.prefill_segmented(prompt, 63 * segment_chunks)
    assert (mono - seg).abs().max().item() <= 2e-4 * mono.abs().max().item()
    assert len(s_seg.chunks) == len(s_mono.chunks) == 6 and s_seg.position == s_mono.position
    for g in range(2):
        a, b = s_mono.chunks.current_retrieved_indices(g), s_seg.chunks.current_retrieved_indices(g)
        assert torch.equal(a[0][:, :b[0].shape[1]], b[0][:, :a[0].shape[1]])
    tok = mono[:, -1].argmax(-1)
    for _ in range(70):                                        # across one chunk boundary
        la, lb = model.decode_step(tok, s_mono), model.decode_step(tok, s_seg)
        assert torch.equal(la.argmax(-1), lb.argmax(-1))
        tok = la.argmax(-1)


@pytest.mark.gpu
def test_training_step_reaches_every_parameter():
    """One bf16 training step at a small shape: the loss is finite and every parameter -- the
    chunk encoder and the K/V projections included, which only the chunk cache connects to the
    loss -- receives a gradient."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    torch.manual_seed(1)
    cfg = D.DRTConfig(hidden_size=256, num_attention_heads=4, intermediate_size=512, vocab_size=1000, decoder_layers=[1, 2],
                      encoder_layers=1, chunk_topk=4, slide_window=128, chunk_id=999)
    model = D.DRTMinimal(cfg).cuda().bfloat16().train()
    tok = torch.randint(0, 999, (2, 63 * 10), device="cuda")
    loss = model(tok, labels=tok)
    assert torch.isfinite(loss)
    loss.backward()
    missing = [n for n, p in model.named_parameters() if p.grad is None or not torch.isfinite(p.grad).all()]
    assert missing == [], missing
    assert model.chunk_k_proj.weight.grad.abs().max().item() > 0
    assert model.encoder[0].mlp.down_proj.weight.grad.abs().max().item() > 0


@pytest.mark.gpu
def test_fused_evaluation_loss_matches_the_unfused_loss():
    """Evaluation (no autograd, bf16) takes the fused norm + LM head + cross-entropy GEMM; the same model
    with autograd on takes the chunked torch path: the two losses must agree to bf16 accuracy."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from long_context_modeling_b200 import drt_minimal as D
    torch.manual_seed(3)
    cfg = D.DRTConfig(hidden_size=128, num_attention_heads=2, intermediate_size=256, decoder_layers=[1, 1], encoder_layers=1,
                      vocab_size=1000, chunk_topk=2, slide_window=32, chunk_id=999)
    model = D.DRTMinimal(cfg).cuda().bfloat16().eval()
    tok = torch.randint(0, 999, (2, 63 * 5), device="cuda")
    with torch.no_grad():
        fused = model(tok, labels=tok)
    unfused = model(tok, labels=tok)                    # autograd on: the chunked torch cross-entropy
    assert abs(fused.item() - unfused.item()) <= 2e-2 * abs(unfused.item()), (fused.item(), unfused.item())


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_graphed_generation_equals_eager_generation(dtype):
    """The CUDA-graph decoder (token steps between chunk boundaries replayed, boundary steps eager) must
    produce exactly the tokens of the eager loop: across two chunk boundaries, starting with a full
    self-attention window."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from long_context_modeling_b200 import drt_minimal as D
    torch.manual_seed(5)
    cfg = D.DRTConfig(hidden_size=128, num_attention_heads=2, intermediate_size=256, decoder_layers=[1, 2], encoder_layers=1,
                      vocab_size=500, chunk_topk=2, slide_window=40, chunk_id=499)
    model = D.DRTMinimal(cfg).cuda().to(dtype).eval()
    prompt = torch.randint(0, 499, (2, 63 * 3), device="cuda")
    eager = model.generate(prompt, 150)
    graphed = model.generate_graphed(prompt, 150)
    assert graphed.shape == eager.shape == (2, 63 * 3 + 150)
    assert torch.equal(graphed, eager)


@pytest.mark.gpu
@pytest.mark.parametrize("virtual", [False, True])
def test_graph_is_reused_across_chunk_boundaries(virtual):
    """The captured token step reads the chunk cache through the view over all backed chunk slots and the
    retrieved ids through static buffers, so one graph serves the spans after later boundaries too: with a
    page-mapped cache (nothing moves) five boundaries need one capture, with the doubling cache a capture
    only follows a re-allocation -- and the tokens stay those of the eager loop."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from long_context_modeling_b200 import drt_minimal as D
    torch.manual_seed(6)
    cfg = D.DRTConfig(hidden_size=128, num_attention_heads=2, intermediate_size=256, decoder_layers=[1, 2], encoder_layers=1,
                      vocab_size=500, chunk_topk=2, slide_window=40, chunk_id=499)
    model = D.DRTMinimal(cfg).cuda().bfloat16().eval()
    prompt = torch.randint(0, 499, (2, 63 * 3), device="cuda")
    new = 330                                                     # five chunk boundaries
    eager = model.generate(prompt, new)
    with torch.no_grad():
        state = D.DecodeState(cfg)
        if virtual:
            import long_context_modeling_b200 as lcm
            state.chunks = lcm.ChunkKVManager(group_size=1, capacity=4, zero_landmark=True, max_chunks=64)
        tok = model(prompt, state=state)[:, -1].argmax(-1)
        dec = D.GraphedDecoder(model, state)
        out = torch.cat([prompt, tok.view(-1, 1), dec.run(tok, new - 1)], dim=1)
    assert torch.equal(out, eager)
    assert dec.captures == 1 if virtual else 1 <= dec.captures <= 3, dec.captures
    if virtual:
        state.chunks.close()


@pytest.mark.gpu
def test_replayed_landmark_step_matches_the_eager_boundary_step():
    """In fused form the decoder closes a chunk without an eager pass over the layers: the chunk's last token
    and then the landmark position are replays of the token-step graph, followed by the chunk encoder, the
    append and the retrieval.  Against ``decode_step`` (one two-position step) from the same state: same cache
    length and position, the appended chunk's K / V / landmark, every cached window and the staged-row state
    equal within bf16 accuracy, and the retrieved chunk ids the same."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import copy
    from long_context_modeling_b200 import drt_minimal as D
    torch.manual_seed(12)
    cfg = D.DRTConfig(hidden_size=128, num_attention_heads=2, intermediate_size=256, decoder_layers=[1, 2], encoder_layers=1,
                      vocab_size=500, chunk_topk=2, slide_window=40, chunk_id=499)
    model = D.DRTMinimal(cfg).cuda().bfloat16().eval()
    prompt = torch.randint(0, 499, (3, 63 * 4), device="cuda")
    forced = torch.randint(0, 499, (3, 63), device="cuda")
    with torch.no_grad():
        state = D.DecodeState(cfg)
        model(prompt, state=state)
        for t in range(62):                                       # up to the chunk's last token, teacher-forced
            model.decode_step(forced[:, t], state)
        assert state.position % model.chunk == 62
        eager, fast = state, copy.deepcopy(state)
        model.decode_step(forced[:, 62], eager)                   # token 62 + landmark, encoder, append, retrieval
        dec = D.GraphedDecoder(model, fast, fused=True)
        assert dec.fused
        dec.run(forced[:, 62].contiguous(), 1)
    assert dec.captures == 1
    assert fast.position == eager.position and len(fast.chunks) == len(eager.chunks) == 5
    assert fast.chunks.lower_hidden_states is None and eager.chunks.lower_hidden_states is None

    def close(a, b, what):
        err, ref = (a.float() - b.float()).abs().max().item(), b.float().abs().max().item()
        assert err <= 3e-2 * ref, (what, err, ref)

    close(fast.chunks.chunk_k[:, -1], eager.chunks.chunk_k[:, -1], "appended K")
    close(fast.chunks.chunk_v[:, -1], eager.chunks.chunk_v[:, -1], "appended V")
    close(fast.chunks.past_lmk_embeds[:, -1], eager.chunks.past_lmk_embeds[:, -1], "appended landmark")
    for li, ((ka, va), (kb, vb)) in enumerate(zip(fast.self_attn, eager.self_attn)):
        close(ka, kb, f"window K of layer {li}")
        close(va, vb, f"window V of layer {li}")
    ia, wa = fast.chunks.current_retrieved_indices(0)
    ib, wb = eager.chunks.current_retrieved_indices(0)
    assert torch.equal(ia.sort(-1).values, ib.sort(-1).values)
    close(wa.sort(-1).values, wb.sort(-1).values, "retrieval weights")


@pytest.mark.gpu
def test_flash_attn_path_matches_torch_path():
    """Where the flash-attn library loads, the body's windowed ALiBi self-attention goes through it (as in the
    reference); the block-banded torch path is the fallback.  Both must agree in bf16: a full sequence, and a
    later segment whose queries sit behind the cached window."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from long_context_modeling_b200 import drt_minimal as D
    if D._flash_attn_func is None:
        pytest.skip("flash-attn is not loadable here")
    torch.manual_seed(2)
    cfg = D.DRTConfig(hidden_size=128, num_attention_heads=2, intermediate_size=256, slide_window=48)
    att = D.SelfAttention(cfg).cuda().bfloat16()
    x = torch.randn(2, 200, 128, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        o_fa, cache = att(x, use_cache=True)
        seg_fa, _ = att(x[:, :70], cache=cache)
        saved, D._flash_attn_func = D._flash_attn_func, None
        try:
            o_t, cache_t = att(x, use_cache=True)
            seg_t, _ = att(x[:, :70], cache=cache_t)
        finally:
            D._flash_attn_func = saved
    assert (o_fa.float() - o_t.float()).abs().max().item() <= 2e-2 * o_t.float().abs().max().item()
    assert (seg_fa.float() - seg_t.float()).abs().max().item() <= 2e-2 * seg_t.float().abs().max().item()


@pytest.mark.gpu
def test_fused_token_step_matches_the_module_path():
    """The graphed decoder's fused token step (norm folded into one q|k|v and one gate|up GEMM, residual adds in
    the o_proj / down_proj epilogues, the library's windowed decode attention and fused GCA sub-layer) against the
    same step through the unfused modules: same state, same token, logits within bf16 accuracy -- and a whole
    graphed generation in fused form runs and keeps the device status clean."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import long_context_modeling_b200 as lcm
    from long_context_modeling_b200 import drt_minimal as D
    torch.manual_seed(9)
    cfg = D.DRTConfig(hidden_size=128, num_attention_heads=2, intermediate_size=256, decoder_layers=[1, 2], encoder_layers=1,
                      vocab_size=500, chunk_topk=2, slide_window=40, chunk_id=499)
    model = D.DRTMinimal(cfg).cuda().bfloat16().eval()
    prompt = torch.randint(0, 499, (3, 63 * 3), device="cuda")
    hidden = []
    with torch.no_grad():
        for fused in (False, True):
            state = D.DecodeState(cfg)
            tok = model(prompt, state=state)[:, -1].argmax(-1)
            dec = D.GraphedDecoder(model, state, fused=fused)
            assert dec.fused == fused
            assert dec._window_full()
            dec.tok = tok.clone()
            dec.stage = torch.zeros(3, model.chunk, 128, dtype=torch.bfloat16, device="cuda")
            dec._make_counters("cuda")
            dec._bind_inputs()
            steps = []
            for t in range(3):                                   # three consecutive token steps, teacher-forced
                steps.append(model.logits(dec._hidden_fused() if fused else dec._hidden_plain()).float())
                dec.tok.copy_(prompt[:, t])
                dec.counters += 1
            hidden.append(torch.stack(steps))
        a, b = hidden
        assert (a - b).abs().max().item() <= 3e-2 * a.abs().max().item(), ((a - b).abs().max().item(), a.abs().max().item())
        out = model.generate_graphed(prompt, 100, fused=True)
    assert out.shape == (3, 63 * 3 + 100)
    assert lcm.read_status() == 0
