"""Decode-step kernels and the CUDA-graph beam decoder against the step-by-step reference path."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _model(layers=2, emb=128, heads=2, vocab=512, sharp=False):
  from t5x_b200 import adafactor, models, trainer as trainer_lib
  from t5x_b200.data import vocabularies
  from t5x_b200.models.t5 import network
  cfg = network.T5Config(vocab_size=vocab, dtype="bfloat16", emb_dim=emb, num_heads=heads,
                         num_encoder_layers=layers, num_decoder_layers=layers, head_dim=64,
                         mlp_dim=256, mlp_activations=("gelu", "linear"), dropout_rate=0.0,
                         logits_via_embedding=not sharp)
  torch.manual_seed(5)
  module = network.Transformer(cfg, device=torch.device("cuda"))
  if sharp:
    with torch.no_grad():
      # sharper next-token distributions than a random initialisation gives: near-ties between
      # candidates would otherwise let bf16 rounding differences reorder the beams
      module.decoder.logits_dense.kernel.mul_(8.0)
  v = vocabularies.PassThroughVocabulary(vocab)
  model = models.EncoderDecoderModel(module, v, v, adafactor.Adafactor())
  from t5x_b200.models import base
  trainer_lib.attach_compute_buffers(base.module_param_tree(module), bf16_copy=True,
                                     main_grad=False)
  return model


def test_decode_self_attention_matches_dense_attention():
  from t5x_b200 import decoding_fast
  torch.manual_seed(0)
  b, k, L, H, D = 3, 4, 24, 2, 64
  rows = b * k
  cache_k = torch.zeros(b, k, H, L, D, device="cuda", dtype=torch.bfloat16)
  cache_v = torch.zeros_like(cache_k)
  # a history in which every position of a beam lives in some other slot
  hist_k = torch.randn(b, k, L, H, D, device="cuda").bfloat16()
  hist_v = torch.randn(b, k, L, H, D, device="cuda").bfloat16()
  anc = torch.randint(0, k, (b, k, L), device="cuda", dtype=torch.int32)
  cur = 17
  for bb in range(b):
    for j in range(k):
      for t in range(cur):
        cache_k[bb, anc[bb, j, t], :, t] = hist_k[bb, anc[bb, j, t], t]
        cache_v[bb, anc[bb, j, t], :, t] = hist_v[bb, anc[bb, j, t], t]
  qkv = torch.randn(rows, 3, H, D, device="cuda").bfloat16()
  bias = torch.randn(H, L, device="cuda")
  out = torch.empty(rows, H, D, device="cuda", dtype=torch.bfloat16)
  cur_t = torch.tensor([cur], device="cuda", dtype=torch.int32)
  decoding_fast.decode_self_attention(qkv[:, 0], qkv[:, 1], qkv[:, 2], cache_k, cache_v, anc,
                                      bias, cur_t, out, k)
  torch.cuda.synchronize()
  # dense oracle in fp32
  for r in range(rows):
    bb, j = divmod(r, k)
    ks = torch.stack([cache_k[bb, anc[bb, j, t], :, t] for t in range(cur)] + [qkv[r, 1]]).float()
    vs = torch.stack([cache_v[bb, anc[bb, j, t], :, t] for t in range(cur)] + [qkv[r, 2]]).float()
    s = torch.einsum("hd,thd->ht", qkv[r, 0].float(), ks) + bias[:, :cur + 1]
    o = torch.einsum("ht,thd->hd", torch.softmax(s, -1), vs)
    assert (out[r].float() - o).abs().max() < 3e-2
  # the new key/value were appended to the row's own slot
  for r in range(rows):
    bb, j = divmod(r, k)
    assert torch.equal(cache_k[bb, j, :, cur], qkv[r, 1]) and \
        torch.equal(cache_v[bb, j, :, cur], qkv[r, 2])


def test_decode_cross_attention_matches_dense_attention():
  from t5x_b200 import decoding_fast
  torch.manual_seed(2)
  b, beams, lk, H, D = 3, 4, 100, 2, 64
  q = torch.randn(b * beams, H, D, device="cuda").bfloat16()
  k = torch.randn(b, lk, H, D, device="cuda").bfloat16()
  v = torch.randn(b, lk, H, D, device="cuda").bfloat16()
  mask = torch.ones(b, lk, dtype=torch.uint8, device="cuda")
  mask[1, 60:] = 0
  out = torch.empty_like(q)
  decoding_fast.decode_cross_attention(q, k.transpose(1, 2).contiguous(),
                                       v.transpose(1, 2).contiguous(), mask, out, beams)
  torch.cuda.synchronize()
  qf = q.float().view(b, beams, H, D)
  s = torch.einsum("bjhd,bthd->bhjt", qf, k.float())
  s = s + (1.0 - mask.float())[:, None, None, :] * -1e10
  o = torch.einsum("bhjt,bthd->bjhd", torch.softmax(s, -1), v.float()).reshape(b * beams, H, D)
  assert (out.float() - o).abs().max() < 3e-2


@pytest.mark.parametrize("shape", [(256, 2048, 2048, 4), (256, 2048, 5120, 5), (64, 512, 1024, 8)])
def test_gemm_splitk(shape):
  from t5x_b200.ops import native
  M, N, K, S = shape
  torch.manual_seed(3)
  a = torch.randn(M, K, device="cuda").bfloat16()
  w = (torch.randn(K, N, device="cuda") * 0.05).bfloat16()
  r = torch.randn(M, N, device="cuda").bfloat16()
  ref = a.float() @ w.float()
  out = native.gemm_splitk(a, w, S)
  out_r = native.gemm_splitk(a, w, S, residual=r)
  native.check_status()
  scale = ref.abs().max()
  assert (out.float() - ref).abs().max() / scale < 1e-2
  assert (out_r.float() - (ref + r.float())).abs().max() / scale < 2e-2
  # a shared workspace that starts clear stays clear: two GEMMs back to back, no fill between
  ws = torch.zeros(M * N + 64, dtype=torch.float32, device="cuda")
  first = native.gemm_splitk(a, w, S, workspace=ws, workspace_is_clear=True)
  second = native.gemm_splitk(a, w, S, residual=r, workspace=ws, workspace_is_clear=True)
  native.check_status()
  assert float(ws.abs().max()) == 0.0
  assert (first.float() - ref).abs().max() / scale < 1e-2
  assert (second.float() - (ref + r.float())).abs().max() / scale < 2e-2


@pytest.mark.parametrize("m,k,n,splits,transposed,with_res", [
    (256, 2048, 2048, None, False, True), (256, 5120, 2048, None, False, True),
    (64, 512, 1024, 8, False, False), (200, 1024, 256, 4, False, True),
    (256, 2048, 2048, 1, False, True), (128, 256, 128, 2, True, True),
    (37, 128, 384, 2, True, False), (256, 2048, 2048, 2, False, False)])
def test_gemm_skinny_cluster_split_k(m, k, n, splits, transposed, with_res):
  """The cluster split-K GEMM (partial products added through distributed shared memory)
  against an fp32 matmul, for every cluster size, both weight layouts and a row tail."""
  from t5x_b200.ops import native
  torch.manual_seed(m + k + n)
  a = torch.randn(m, k, device="cuda").bfloat16()
  if transposed:
    w = (torch.randn(n, k, device="cuda") * 0.05).bfloat16().t()
  else:
    w = (torch.randn(k, n, device="cuda") * 0.05).bfloat16()
  res = torch.randn(m, n, device="cuda").bfloat16() if with_res else None
  if splits is None:
    assert native.gemm_skinny_splits(m, n, k) in (2, 4, 8)
  out = native.gemm_skinny(a, w, residual=res, splits=splits)
  assert out is not None
  native.check_status()
  ref = a.float() @ w.float()
  if res is not None:
    ref = ref + res.float()
  err = (out.float() - ref).abs().max() / ref.abs().max()
  assert err < 8e-3, err
  # twice in a row over the same buffers: nothing is left behind between launches
  out2 = native.gemm_skinny(a, w, residual=res, splits=splits)
  assert torch.equal(out, out2)


def test_gemm_skinny_declines_shapes_it_does_not_cover():
  from t5x_b200.ops import native
  assert native.gemm_skinny_splits(256, 2000, 2048) == 0     # N % 128
  assert native.gemm_skinny_splits(256, 2048, 2000) == 0     # K % 64
  assert native.gemm_skinny_splits(4096, 32128 // 128 * 128, 2048) == 0  # more tiles than SMs
  a = torch.randn(16, 100, device="cuda").bfloat16()
  w = torch.randn(100, 128, device="cuda").bfloat16()
  assert native.gemm_skinny(a, w) is None


@pytest.mark.parametrize("use_graph", [False, True])
def test_graph_beam_decoder_matches_reference_beam_search(use_graph):
  from t5x_b200 import decoding_fast
  model = _model()
  torch.manual_seed(1)
  b, le, ld, beams = 3, 32, 12, 4
  enc = torch.randint(2, 512, (b, le), device="cuda")
  enc[1, 20:] = 0
  batch = {"encoder_input_tokens": enc,
           "decoder_input_tokens": torch.zeros(b, ld, dtype=torch.long, device="cuda")}
  os.environ["T5X_B200_GRAPH_DECODE"] = "0"
  try:
    ref_seqs, ref_aux = model.predict_batch_with_aux(None, batch, return_all_decodes=True,
                                                     num_decodes=beams)
  finally:
    os.environ.pop("T5X_B200_GRAPH_DECODE")
  dec = decoding_fast.GraphBeamDecoder(model.module, b, beams, ld, eos_id=1, alpha=0.6,
                                       use_graph=use_graph)
  for _ in range(2):  # second call reuses the captured graph
    seqs, scores = dec.decode(enc)
  assert seqs.shape == ref_seqs.shape and scores.shape == ref_aux["scores"].shape
  # bf16 kernels differ between the two paths; near-ties may reorder, so compare the best beam
  # exactly and all scores loosely
  torch.testing.assert_close(scores[:, -1], ref_aux["scores"][:, -1], rtol=2e-2, atol=5e-2)
  agree = (seqs[:, -1] == ref_seqs[:, -1]).float().mean()
  assert agree > 0.9, (seqs[:, -1], ref_seqs[:, -1])


@pytest.mark.parametrize("beams", [1, 2, 8])
def test_graph_beam_decoder_at_other_beam_widths(beams):
  from t5x_b200 import decoding_fast
  model = _model(sharp=True)
  torch.manual_seed(2)
  b, le, ld = 4, 24, 10
  enc = torch.randint(2, 512, (b, le), device="cuda")
  enc[2, 11:] = 0
  batch = {"encoder_input_tokens": enc,
           "decoder_input_tokens": torch.zeros(b, ld, dtype=torch.long, device="cuda")}
  os.environ["T5X_B200_GRAPH_DECODE"] = "0"
  try:
    ref_seqs, ref_aux = model.predict_batch_with_aux(None, batch, return_all_decodes=True,
                                                     num_decodes=beams)
  finally:
    os.environ.pop("T5X_B200_GRAPH_DECODE")
  dec = decoding_fast.GraphBeamDecoder(model.module, b, beams, ld, eos_id=1, alpha=0.6)
  seqs, scores = dec.decode(enc)
  assert seqs.shape == ref_seqs.shape == (b, beams, ld)
  torch.testing.assert_close(scores[:, -1], ref_aux["scores"][:, -1], rtol=2e-2, atol=0.15)
  # the two paths round differently (bf16 kernels): where the best hypotheses differ, they must
  # be a near-tie, and most examples must agree outright
  same = (seqs[:, -1] == ref_seqs[:, -1]).all(dim=1)
  gap = (scores[:, -1] - ref_aux["scores"][:, -1]).abs()
  assert bool(((same) | (gap < 0.1)).all()), (seqs[:, -1], ref_seqs[:, -1], gap)
  assert int(same.sum()) >= b // 2, (seqs[:, -1], ref_seqs[:, -1])


def test_termination_check_period_changes_when_the_loop_ends_not_what_it_returns():
  """The host looks at the device's 'all batches finished' flag every `period` steps only.
  With an end-of-sequence id that the model emits early, a short period leaves the loop
  sooner; the hypotheses and scores are those of a run that never looks."""
  from t5x_b200 import decoding_fast
  model = _model(sharp=True)
  torch.manual_seed(3)
  b, le, ld, beams = 2, 16, 24, 4
  enc = torch.randint(2, 512, (b, le), device="cuda")
  probe = decoding_fast.GraphBeamDecoder(model.module, b, beams, ld, eos_id=1, alpha=0.6,
                                         termination_check_period=10 ** 6)
  seqs, _ = probe.decode(enc)
  early = seqs[:, -1, 1:4].reshape(-1)
  eos = int(torch.mode(early[early > 1]).values)  # a token that it emits early
  runs = {}
  for period in (10 ** 6, 1, 3, 8):
    dec = decoding_fast.GraphBeamDecoder(model.module, b, beams, ld, eos_id=eos, alpha=0.6,
                                         termination_check_period=period)
    out = dec.decode(enc)
    runs[period] = (out, dec.replays)
  (want_seqs, want_scores), full = runs[10 ** 6]
  assert full == ld
  for period in (1, 3, 8):
    (got_seqs, got_scores), n = runs[period]
    assert n <= full and (n == full or n % period == 0)
    torch.testing.assert_close(got_scores, want_scores)
    assert torch.equal(got_seqs, want_seqs)
  assert runs[1][1] <= runs[3][1] + 2 and runs[1][1] <= runs[8][1]


@pytest.mark.parametrize("level", [1, 2])
def test_chained_launches_do_not_change_the_decode(level, monkeypatch):
  """Programmatic dependent launches (each kernel set up behind its predecessor, level 2 also
  requesting the constant weights ahead of the wait) give the same beams and scores."""
  from t5x_b200 import decoding_fast
  model = _model(sharp=True)
  torch.manual_seed(4)
  enc = torch.randint(2, 512, (3, 20), device="cuda")
  plain = decoding_fast.GraphBeamDecoder(model.module, 3, 4, 12, eos_id=1, alpha=0.6)
  want_seqs, want_scores = plain.decode(enc)
  monkeypatch.setenv("T5X_B200_DECODE_CHAIN", str(level))
  chained = decoding_fast.GraphBeamDecoder(model.module, 3, 4, 12, eos_id=1, alpha=0.6)
  assert chained.chain_level == level
  for _ in range(2):  # eager warm-up + capture, then replay
    got_seqs, got_scores = chained.decode(enc)
  from t5x_b200.ops import native
  native.check_status()
  assert torch.equal(got_seqs, want_seqs)
  torch.testing.assert_close(got_scores, want_scores, rtol=1e-4, atol=1e-4)


def test_predict_batch_uses_graph_decoder_by_default():
  model = _model()
  enc = torch.randint(2, 512, (2, 16), device="cuda")
  batch = {"encoder_input_tokens": enc,
           "decoder_input_tokens": torch.zeros(2, 8, dtype=torch.long, device="cuda")}
  out = model.predict_batch(None, batch)
  assert out.shape == (2, 8)
  assert model.__dict__.get("_graph_decoders")


@pytest.mark.parametrize("beams,lk", [(1, 37), (4, 512), (8, 1000), (2, 16)])
def test_decode_cross_attention_on_tensor_cores(beams, lk):
  """The mma.sync cross-attention (permuted channel and key order, transposed values) against
  fp32: every beam of an example attends over that example's keys, padding masked."""
  from t5x_b200 import decoding_fast
  from t5x_b200.ops import native
  torch.manual_seed(beams * 1000 + lk)
  b, H, D = 3, 5, 64
  rows = b * beams
  q = (torch.randn(rows, H, D, device="cuda") * 0.5).bfloat16()
  k = (torch.randn(b, lk, H, D, device="cuda") * 0.5).bfloat16()
  v = torch.randn(b, lk, H, D, device="cuda").bfloat16()
  lens = torch.tensor([lk, max(1, lk // 2), max(1, lk - 3)], device="cuda")
  mask = torch.arange(lk, device="cuda")[None, :] < lens[:, None]
  kp, vt = decoding_fast.cross_kv_layout(k, v)
  out = torch.empty(rows, H, D, device="cuda", dtype=torch.bfloat16)
  decoding_fast.decode_cross_attention_mma(q, kp, vt, mask.to(torch.uint8).contiguous(), out,
                                           beams, lk)
  native.check_status()
  qf = q.float().view(b, beams, H, D)
  s = torch.einsum("bjhd,bthd->bhjt", qf, k.float())
  s = s + torch.where(mask, 0.0, -1e10)[:, None, None, :]
  want = torch.einsum("bhjt,bthd->bjhd", torch.softmax(s, -1), v.float()).reshape(rows, H, D)
  assert (out.float() - want).abs().max() < 3e-2
  # no mask at all
  decoding_fast.decode_cross_attention_mma(q, kp, vt, None, out, beams, lk)
  s = torch.einsum("bjhd,bthd->bhjt", qf, k.float())
  want = torch.einsum("bhjt,bthd->bjhd", torch.softmax(s, -1), v.float()).reshape(rows, H, D)
  assert (out.float() - want).abs().max() < 3e-2


@pytest.mark.parametrize("beams,cur", [(4, 17), (4, 0), (8, 70), (1, 40), (2, 95)])
def test_decode_self_attention_on_tensor_cores(beams, cur):
  """The mma.sync self-attention over the ancestry-indexed cache (transposed value cache, keys
  of all slots multiplied and masked by ownership) against the dense fp32 statement; the new
  key row / value column land in the row's own slot."""
  from t5x_b200 import decoding_fast
  from t5x_b200.ops import native
  torch.manual_seed(beams * 100 + cur)
  b, L, H, D = 3, 100, 2, 64
  lc = -(-L // 32) * 32
  assert decoding_fast.self_mma_supported(beams, L)
  rows = b * beams
  cache_k = torch.zeros(b, beams, H, lc, D, device="cuda", dtype=torch.bfloat16)
  cache_vt = torch.zeros(b, beams, H, D, lc, device="cuda", dtype=torch.bfloat16)
  hist_k = (torch.randn(b, beams, L, H, D, device="cuda") * 0.5).bfloat16()
  hist_v = torch.randn(b, beams, L, H, D, device="cuda").bfloat16()
  # every (slot, position) holds something, also beyond `cur` (stale entries of an earlier
  # decode must not matter); a beam's history at position t lives in slot anc[b, j, t]
  cache_k[:, :, :, :L] = hist_k.permute(0, 1, 3, 2, 4)
  cache_vt[:, :, :, :, :L] = hist_v.permute(0, 1, 3, 4, 2)
  anc = torch.randint(0, beams, (b, beams, L), device="cuda", dtype=torch.int32)
  qkv = (torch.randn(rows, 3, H, D, device="cuda") * 0.5).bfloat16()
  bias = torch.randn(H, L, device="cuda")
  out = torch.empty(rows, H, D, device="cuda", dtype=torch.bfloat16)
  cur_t = torch.tensor([cur], device="cuda", dtype=torch.int32)
  decoding_fast.decode_self_attention_mma(qkv[:, 0], qkv[:, 1], qkv[:, 2], cache_k, cache_vt, anc,
                                          bias, cur_t, out, beams, L)
  native.check_status()
  torch.cuda.synchronize()
  for r in range(rows):
    bb, j = divmod(r, beams)
    ks = torch.stack([hist_k[bb, anc[bb, j, t], t] for t in range(cur)] + [qkv[r, 1]]).float()
    vs = torch.stack([hist_v[bb, anc[bb, j, t], t] for t in range(cur)] + [qkv[r, 2]]).float()
    s = torch.einsum("hd,thd->ht", qkv[r, 0].float(), ks) + bias[:, :cur + 1]
    o = torch.einsum("ht,thd->hd", torch.softmax(s, -1), vs)
    assert (out[r].float() - o).abs().max() < 3e-2, (r, (out[r].float() - o).abs().max())
    assert torch.equal(cache_k[bb, j, :, cur], qkv[r, 1])
    assert torch.equal(cache_vt[bb, j, :, :, cur], qkv[r, 2])
