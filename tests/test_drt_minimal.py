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
