"""Beam search for the T5 encoder-decoder as one replayed CUDA graph per step.

Same algorithm and results as `decoding.beam_search` driven through
`EncoderDecoderModel.predict_batch_with_aux` (t5x/decoding.py:1131-1569, t5x/models.py:584-758)
for decoding without a prompt, restated for the GPU:

* every tensor of the search state is a fixed-size device buffer and the position counter is a
  device scalar, so one decode step (24 decoder layers + the beam bookkeeping) is captured once
  and replayed; the host only reads a termination flag every few steps;
* the self-attention key/value cache is never reordered. Each (batch, beam) row appends its new
  key/value to its own slot, and a small `ancestry[batch, beam, position]` table records which
  slot holds a beam's history; reselecting beams rewrites that table (kilobytes) instead of
  gathering every layer's cache (gigabytes);
* cross-attention keys/values are projected once per example and shared by its beams;
* q/k/v projections of a layer are one GEMM over a concatenated weight.
"""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch

from t5x_b200 import decoding
from t5x_b200.ops import attention as attn_ops
from t5x_b200.ops import native
from t5x_b200.ops import reference as ref

c_void_p, c_int, c_ll = native.c_void_p, native.c_int, native.c_ll
native.register_signature("t5x_decode_self_attention",
                          [c_void_p] * 9 + [c_ll, c_int, c_int, c_int, c_int, c_int, c_void_p])
native.register_signature("t5x_decode_cross_attention",
                          [c_void_p] * 5 + [c_ll, c_int, c_int, c_int, c_int, c_int, c_void_p])
native.register_signature("t5x_decode_self_attention_mma",
                          [c_void_p] * 9 + [c_ll, c_int, c_int, c_int, c_int, c_int, c_int,
                           c_void_p])
native.register_signature("t5x_decode_cross_attention_mma",
                          [c_void_p] * 5 + [c_ll, c_int, c_int, c_int, c_int, c_int, c_int,
                           c_void_p])

NEG_INF = decoding.NEG_INF


def decode_self_attention(q, k_new, v_new, cache_k, cache_v, ancestry, bias_row, cur_index, out,
                          beams: int) -> None:
  """One decode step of self-attention over an ancestry-indexed cache (see csrc/decode.cu)."""
  rows, heads, hd = q.shape
  assert q.stride(2) == 1 and q.stride(1) == hd and k_new.stride() == q.stride() and \
      v_new.stride() == q.stride()
  native._check(native.lib().t5x_decode_self_attention(
      q.data_ptr(), k_new.data_ptr(), v_new.data_ptr(), cache_k.data_ptr(), cache_v.data_ptr(),
      ancestry.data_ptr(), native.ptr(bias_row), cur_index.data_ptr(), out.data_ptr(),
      q.stride(0), rows, beams, heads, hd, cache_k.shape[3], native.stream_ptr()),
      "decode_self_attention")


def self_mma_supported(beams: int, max_len: int) -> bool:
  """Whether `decode_self_attention_mma` covers this search (its chunk budget is 32 chunks of
  32 positions over all beams)."""
  return beams in (1, 2, 4, 8) and beams * (-(-max_len // 32)) <= 32 and max_len <= 1024


def decode_self_attention_mma(q, k_new, v_new, cache_k, cache_vt, ancestry, bias_row, cur_index,
                              out, beams: int, max_len: int) -> None:
  """One decode step of self-attention over an ancestry-indexed cache on the tensor cores
  (csrc/decode_self_mma.cu): cache_k [b, beams, H, Lc, 64], cache_vt [b, beams, H, 64, Lc]."""
  rows, heads, hd = q.shape
  lc = cache_k.shape[3]
  assert q.stride(2) == 1 and q.stride(1) == hd and k_new.stride() == q.stride() and \
      v_new.stride() == q.stride()
  assert cache_k.is_contiguous() and cache_vt.is_contiguous() and cache_vt.shape[4] == lc
  native._check(native.lib().t5x_decode_self_attention_mma(
      q.data_ptr(), k_new.data_ptr(), v_new.data_ptr(), cache_k.data_ptr(), cache_vt.data_ptr(),
      ancestry.data_ptr(), native.ptr(bias_row), cur_index.data_ptr(), out.data_ptr(),
      q.stride(0), rows // beams, beams, heads, hd, max_len, lc, native.stream_ptr()),
      "decode_self_attention_mma")


def decode_cross_attention(q, k, v, key_mask_u8, out, beams: int) -> None:
  """`beams` query rows per example against that example's encoder keys/values."""
  rows, heads, hd = q.shape
  b, lk = k.shape[0], k.shape[2]  # k, v: [batch, heads, Lk, 64]
  assert k.is_contiguous() and v.is_contiguous() and q.stride(2) == 1 and q.stride(1) == hd
  native._check(native.lib().t5x_decode_cross_attention(
      q.data_ptr(), k.data_ptr(), v.data_ptr(), native.ptr(key_mask_u8), out.data_ptr(),
      q.stride(0), b, beams, heads, hd, lk, native.stream_ptr()), "decode_cross_attention")


def _register_tp_signatures():
  import ctypes
  pp = ctypes.POINTER(c_void_p)
  native.register_signature("t5x_decode_step_advance", [c_void_p, c_void_p])
  native.register_signature("t5x_decode_push_partial",
                            [c_void_p, c_ll, pp, pp, c_int, c_int, c_void_p, c_void_p, c_void_p])
  native.register_signature("t5x_decode_sum_slots",
                            [c_void_p, c_int, c_int, c_ll, c_void_p, c_void_p, c_void_p, c_void_p,
                             c_void_p])
  native.register_signature("t5x_decode_sum_slots_norm",
                            [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                             native.c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p])
  native.register_signature("t5x_decode_gather_push",
                            [c_void_p, c_int, c_int, c_int, c_int, pp, pp, c_int, c_int, c_void_p,
                             c_void_p, c_void_p])
  native.register_signature("t5x_decode_wait", [c_void_p, c_int, c_int, c_void_p, c_void_p])


class _TensorParallelLink:
  """Peer-memory plumbing of a tensor-parallel decode step (kernels in csrc/decode_tp.cu).

  Weights are sharded over the model axis as in training (heads, mlp and vocab), the
  activations [rows, d_model] are replicated. Every row-parallel projection of the step (three
  per layer) is an all-reduce site with an inbox and a row of signal words of its own on every
  rank, numbered in the order the step reaches them; the logits are one more site, a gather
  of vocabulary slices. The epoch that the signals carry is a step counter in device memory,
  advanced by the step itself, so the step can be captured in a CUDA graph and replayed."""

  def __init__(self, group, rows: int, width: int, sites: int, vocab: int, device):
    from t5x_b200.ops import comm
    _register_tp_signatures()
    self.comm = comm
    self.rows, self.width, self.sites, self.vocab = rows, width, sites, vocab
    self.n = rows * width
    if self.n % 8 or vocab % 4:
      raise ValueError("tensor-parallel decode wants rows * d_model % 8 == 0 and vocab % 4 == 0")
    import torch.distributed as dist
    self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
    self.inbox = comm.SymmetricBuffer(sites * self.world * self.n, torch.float32, group, device)
    self.logits = comm.SymmetricBuffer(rows * vocab, torch.float32, group, device)
    self.sig = comm.SymmetricBuffer((sites + 1) * 16, torch.int32, group, device)
    self.sig.tensor.zero_()
    self.step = torch.zeros(1, dtype=torch.int32, device=device)
    self.ticket = torch.zeros(1, dtype=torch.int32, device=device)
    self.ws = torch.zeros(self.n, dtype=torch.float32, device=device)
    torch.cuda.synchronize(device)
    dist.barrier(group=group)  # every rank's signal words are zero before anyone raises one
    self.site = 0

  def begin_step(self) -> None:
    native._check(native.lib().t5x_decode_step_advance(self.step.data_ptr(), native.stream_ptr()),
                  "decode_step_advance")
    self.site = 0

  def _sig_ptrs(self, site: int):
    return self.comm._ptr_array([p + site * 16 * 4 for p in self.sig.peer_ptrs])

  def all_reduce(self, a: torch.Tensor, w: torch.Tensor, residual: torch.Tensor, splits: int,
                 norm_scale: Optional[torch.Tensor] = None, eps: float = 1e-6):
    """x = sum over ranks of (a @ w) + residual, bf16 [rows, width], identical on every rank.
    With `norm_scale` returns (x, rmsnorm(x) * norm_scale) from one kernel."""
    site = self.site
    self.site += 1
    assert site < self.sites
    ws = self.ws.view(self.rows, self.width)
    native.gemm_splitk_accumulate(a, w, ws, max(1, splits), accumulate=True)
    slot_bytes = self.n * 4
    base = site * self.world * slot_bytes + self.rank * slot_bytes
    slots = self.comm._ptr_array([p + base for p in self.inbox.peer_ptrs])
    native._check(native.lib().t5x_decode_push_partial(
        self.ws.data_ptr(), self.n, slots, self._sig_ptrs(site), self.world, self.rank,
        self.step.data_ptr(), self.ticket.data_ptr(), native.stream_ptr()), "decode_push_partial")
    out = torch.empty(self.rows, self.width, dtype=torch.bfloat16, device=a.device)
    inbox = self.inbox.tensor.data_ptr() + site * self.world * slot_bytes
    sig = self.sig.tensor.data_ptr() + site * 16 * 4
    if norm_scale is not None and self.width % 4 == 0 and self.width <= 8192:
      normed = torch.empty_like(out)
      native._check(native.lib().t5x_decode_sum_slots_norm(
          inbox, self.world, self.rank, self.rows, self.width, native.ptr(residual),
          norm_scale.data_ptr(), float(eps), out.data_ptr(), normed.data_ptr(), sig,
          self.step.data_ptr(), native.stream_ptr()), "decode_sum_slots_norm")
      return out, normed
    native._check(native.lib().t5x_decode_sum_slots(
        inbox, self.world, self.rank, self.n, native.ptr(residual), out.data_ptr(), sig,
        self.step.data_ptr(), native.stream_ptr()), "decode_sum_slots")
    if norm_scale is not None:
      return out, native.rmsnorm_fwd(out, norm_scale, eps)[0]
    return out

  def gather_logits(self, local: torch.Tensor) -> torch.Tensor:
    """local [rows, vocab / world] fp32 -> the full [rows, vocab] logits on every rank."""
    site = self.sites  # the last row of signal words
    cols = local.shape[1]
    assert local.is_contiguous() and cols * self.world == self.vocab
    fulls = self.comm._ptr_array(self.logits.peer_ptrs)
    native._check(native.lib().t5x_decode_gather_push(
        local.data_ptr(), self.rows, cols, self.vocab, self.rank * cols, fulls,
        self._sig_ptrs(site), self.world, self.rank, self.step.data_ptr(),
        self.ticket.data_ptr(), native.stream_ptr()), "decode_gather_push")
    native._check(native.lib().t5x_decode_wait(
        self.sig.tensor.data_ptr() + site * 16 * 4, self.world, self.rank, self.step.data_ptr(),
        native.stream_ptr()), "decode_wait")
    return self.logits.tensor.view(self.rows, self.vocab)


def cross_kv_layout(k: torch.Tensor, v: torch.Tensor):
  """(keys [b, H, Lp, 64], values transposed [b, H, 64, Lp]) for `decode_cross_attention_mma`
  from k, v [b, Lk, H, 64]; Lp = Lk rounded up to a multiple of 32, the padding is zero."""
  b, lk, h, d = k.shape
  lp = -(-lk // 32) * 32
  kp = torch.zeros(b, h, lp, d, dtype=k.dtype, device=k.device)
  kp[:, :, :lk] = k.transpose(1, 2)
  vt = torch.zeros(b, h, d, lp, dtype=v.dtype, device=v.device)
  vt[:, :, :, :lk] = v.permute(0, 2, 3, 1)
  return kp, vt


def decode_cross_attention_mma(q, k_padded, v_transposed, key_mask_u8, out, beams: int,
                               lk: int) -> None:
  """`beams` query rows per example against that example's encoder keys / values on the tensor
  cores (csrc/decode_cross_mma.cu); operands as made by `cross_kv_layout`."""
  rows, heads, hd = q.shape
  b, lp = k_padded.shape[0], k_padded.shape[2]
  assert k_padded.is_contiguous() and v_transposed.is_contiguous()
  assert v_transposed.shape == (b, heads, hd, lp) and q.stride(2) == 1 and q.stride(1) == hd
  native._check(native.lib().t5x_decode_cross_attention_mma(
      q.data_ptr(), k_padded.data_ptr(), v_transposed.data_ptr(), native.ptr(key_mask_u8),
      out.data_ptr(), q.stride(0), b, beams, heads, hd, lk, lp, native.stream_ptr()),
      "decode_cross_attention_mma")


def _splits(k_dim: int, n_dim: int, rows: int) -> int:
  """K slices for a skinny GEMM so that about one CTA per SM streams the weights."""
  tiles = -(-rows // 128) * -(-n_dim // 128)
  best = 1
  for s in (2, 4, 5, 8, 10):
    if k_dim % s == 0 and (k_dim // s) % 64 == 0 and tiles * s <= 192:
      best = s
  return best


def supported(module, decoder_input_tokens: torch.Tensor, decode_fn) -> bool:
  """True when `GraphBeamDecoder` covers this model / call."""
  from t5x_b200.models.t5 import network
  from t5x_b200.parallel import state as pstate
  if not isinstance(module, network.Transformer) or decode_fn is not decoding.beam_search:
    return False
  c = module.config
  p = module.token_embedder.embedding
  st = pstate.get()
  zctx = getattr(getattr(p, "zero", None), "ctx", None)
  if zctx is not None and getattr(zctx, "shard_weights", False):
    return False  # layer weights live on their owners; the module's own forward gathers them
  if st.model_size > 1:
    # tensor-parallel decode: heads, mlp and vocabulary split evenly, logits not tied
    import torch.distributed as dist
    if not (dist.is_initialized() and c.num_heads % st.model_size == 0 and
            c.vocab_size % (4 * st.model_size) == 0 and c.emb_dim % 8 == 0 and
            not c.logits_via_embedding and st.model_size <= 16):
      return False
  return (p.is_cuda and getattr(p, "bf16", None) is not None and c.head_dim == 64 and
          tuple(c.mlp_activations) == ("gelu", "linear") and
          decoder_input_tokens.shape[1] + 1 <= 1024 and not c.scale_attn_logits and
          not c.float32_attention_logits)


class _Layer:
  """bf16 weights of one decoder layer, q/k/v concatenated."""

  def __init__(self, layer):
    w = lambda dense: dense.kernel.bf16
    sa, ca, mlp = layer.self_attention, layer.encoder_decoder_attention, layer.mlp
    self.qkv = torch.cat([w(sa.query), w(sa.key), w(sa.value)], dim=1).contiguous()
    self.o = w(sa.out)
    self.cq, self.co = w(ca.query), w(ca.out)
    self.ck, self.cv = w(ca.key), w(ca.value)
    self.wi0, self.wi1, self.wo = w(mlp.wi_0), w(mlp.wi_1), w(mlp.wo)
    self.ln1 = layer.pre_self_attention_layer_norm.scale
    self.ln2 = layer.pre_cross_attention_layer_norm.scale
    self.ln3 = layer.pre_mlp_layer_norm.scale


class GraphBeamDecoder:
  """Static-shape beam search over a `models.t5.network.Transformer`."""

  def __init__(self, module, batch: int, beams: int, max_decode_len: int, eos_id: int,
               alpha: float = 0.6, termination_check_period: int = 8, use_graph: bool = True):
    c = module.config
    self.module, self.c = module, c
    self.b, self.k, self.eos, self.alpha = batch, beams, eos_id, alpha
    self.L = max_decode_len + 1  # position 0 is the dummy BOS
    self.rows = batch * beams
    from t5x_b200.parallel import state as pstate
    st = pstate.get()
    self.tp = st.model_size
    self.H, self.D = c.num_heads // self.tp, c.head_dim  # heads held by this rank
    import os
    self.check_period = max(1, int(os.environ.get("T5X_B200_DECODE_CHECK_PERIOD",
                                                  termination_check_period)))
    self.replays = 0           # graph replays so far
    # programmatic dependent launches inside the step (`native.chained_launches`); the
    # tensor-parallel step keeps ordinary launches: its kernels wait for other ranks
    self.chain_level = int(os.environ.get("T5X_B200_DECODE_CHAIN", "0")) if self.tp == 1 else 0
    # residual projections through the cluster split-K GEMM (sum over K slices in distributed
    # shared memory) instead of fp32 atomics into a workspace plus a finishing kernel
    self.cluster_gemm = os.environ.get("T5X_B200_DECODE_CLUSTER_GEMM", "1") != "0"
    self.kernels_per_step = 0  # this library's kernels inside one captured step
    self.use_graph = use_graph
    dev = module.token_embedder.embedding.device
    self.dev = dev
    dec = module.decoder
    self.layers = [_Layer(getattr(dec, f"layers_{i}")) for i in range(c.num_decoder_layers)]
    self.emb = module.token_embedder.embedding.bf16
    self.link: Optional[_TensorParallelLink] = None
    if self.tp > 1:
      import torch.distributed as dist
      # token lookups need the whole (vocabulary-sharded) table: gathered once, 2 bytes a weight
      parts = [torch.empty_like(self.emb) for _ in range(self.tp)]
      dist.all_gather(parts, self.emb.contiguous(), group=st.model_group)
      self.emb = torch.cat(parts, dim=0)
      self.link = _TensorParallelLink(st.model_group, self.rows, c.emb_dim,
                                      3 * c.num_decoder_layers, c.vocab_size, dev)
    self.final_ln = dec.decoder_norm.scale
    w, self.logit_scale = dec.logits_weight_and_scale()
    wl = w.bf16
    self.w_logits = wl if wl.shape[0] == c.emb_dim else wl.t()
    self.rel_table = dec.relpos_bias.rel_embedding
    bf = dict(dtype=torch.bfloat16, device=dev)
    # [batch, beam slot, head, position, dim]: one (slot, head) history is contiguous. For the
    # tensor-core kernel the cache is padded to a multiple of 32 positions and the values are
    # kept transposed ([..., dim, position]).
    # measured slower than the one-warp-per-row kernel (95 against 75 us per layer at the XL
    # decode shape: the work of an example and head does not fill a CTA of eight warps), so it
    # is opt-in
    self.self_mma = self_mma_supported(beams, self.L) and \
        os.environ.get("T5X_B200_DECODE_SELF_MMA", "0") == "1"
    if self.self_mma:
      lc = -(-self.L // 32) * 32
      self.cache_k = [torch.zeros(batch, beams, self.H, lc, self.D, **bf) for _ in self.layers]
      self.cache_v = [torch.zeros(batch, beams, self.H, self.D, lc, **bf) for _ in self.layers]
    else:
      self.cache_k = [torch.zeros(batch, beams, self.H, self.L, self.D, **bf)
                      for _ in self.layers]
      self.cache_v = [torch.zeros(batch, beams, self.H, self.L, self.D, **bf)
                      for _ in self.layers]
    self.cross_k: List[Optional[torch.Tensor]] = [None] * len(self.layers)
    self.cross_v: List[Optional[torch.Tensor]] = [None] * len(self.layers)
    self.enc_mask = None
    self.enc_mask_u8 = None
    self._ws = None
    i64 = dict(dtype=torch.int64, device=dev)
    self.cur = torch.zeros(1, dtype=torch.int32, device=dev)
    self.live_seqs = torch.zeros(batch, beams, self.L, **i64)
    self.fin_seqs = torch.zeros(batch, beams, self.L, **i64)
    self.live_lp = torch.zeros(batch, beams, device=dev)
    self.fin_scores = torch.zeros(batch, beams, device=dev)
    self.fin_flags = torch.zeros(batch, beams, dtype=torch.bool, device=dev)
    self.anc = torch.zeros(batch, beams, self.L, dtype=torch.int32, device=dev)
    self.terminated = torch.zeros(1, dtype=torch.bool, device=dev)
    self.positions = torch.arange(self.L, device=dev)
    self.min_brevity = float(decoding.brevity_penalty(alpha, self.L))
    self.graph: Optional[torch.cuda.CUDAGraph] = None
    self._graph_enc_len = -1
    self._beam_scratch = None

  # ------------------------------------------------------------------------------------------
  def _reset(self):
    self.cur.zero_()
    self.live_seqs.zero_()
    self.fin_seqs.zero_()
    self.live_lp.copy_(torch.tensor([0.0] + [NEG_INF] * (self.k - 1), device=self.dev)
                       .expand(self.b, self.k))
    self.fin_scores.fill_(NEG_INF)
    self.fin_flags.zero_()
    self.anc.copy_(torch.arange(self.k, dtype=torch.int32, device=self.dev)[None, :, None]
                   .expand(self.b, self.k, self.L))
    self.terminated.zero_()

  def _encode(self, encoder_input_tokens: torch.Tensor):
    enc = self.module.encode(encoder_input_tokens, enable_dropout=False)
    b, le, _ = enc.shape
    flat = enc.reshape(b * le, -1)
    self.enc_len = le
    self.cross_mma = self.k in (1, 2, 4, 8) and le <= 1024
    for i, ly in enumerate(self.layers):
      k = native.gemm(flat, ly.ck).view(b, le, self.H, self.D)
      v = native.gemm(flat, ly.cv).view(b, le, self.H, self.D)
      if self.cross_mma:
        # keys head-major and padded to 16, values transposed: the layouts the tensor-core
        # decode kernel loads straight into its operand registers
        self.cross_k[i], self.cross_v[i] = cross_kv_layout(k, v)
      else:
        self.cross_k[i] = k.transpose(1, 2).contiguous()
        self.cross_v[i] = v.transpose(1, 2).contiguous()
    self.enc_mask = (encoder_input_tokens > 0)
    self.enc_mask_u8 = self.enc_mask.to(torch.uint8).contiguous()
    if self.tp > 1:
      from t5x_b200.parallel import tp_fused
      tp_fused.end_step()  # the encoder pass is over: its arena blocks are free again

  def _model_step(self) -> torch.Tensor:
    """Logits [rows, vocab] (fp32) of the token at position `cur` of every live beam."""
    c, rows, H, D = self.c, self.rows, self.H, self.D
    ci = self.cur.long()
    tok = self.live_seqs.gather(2, ci.view(1, 1, 1).expand(self.b, self.k, 1)).reshape(rows)
    x = self.emb.index_select(0, tok)
    rel = self.positions - ci  # key position minus query position
    buckets = ref.relative_position_bucket(rel, False, c.relpos_num_buckets,
                                           c.relpos_max_distance)
    bias_row = self.rel_table.float()[:, buckets].contiguous()  # [H, L]
    ctx = torch.empty(rows, H, D, dtype=torch.bfloat16, device=self.dev)
    if self.link is not None:
      self.link.begin_step()
    norms = [(ly.ln1, ly.ln2, ly.ln3) for ly in self.layers]
    h, _ = native.rmsnorm_fwd(x, norms[0][0], 1e-6)
    for i, ly in enumerate(self.layers):
      # every residual projection is followed by a norm: `_row_parallel` returns both the new
      # residual stream and its normed form (one finishing kernel on the single-GPU path)
      next_ln1 = norms[i + 1][0] if i + 1 < len(self.layers) else self.final_ln
      qkv = native.gemm(h, ly.qkv).view(rows, 3, H, D)
      if self.self_mma:
        decode_self_attention_mma(qkv[:, 0], qkv[:, 1], qkv[:, 2], self.cache_k[i],
                                  self.cache_v[i], self.anc, bias_row, self.cur, ctx, self.k,
                                  self.L)
      else:
        decode_self_attention(qkv[:, 0], qkv[:, 1], qkv[:, 2], self.cache_k[i], self.cache_v[i],
                              self.anc, bias_row, self.cur, ctx, self.k)
      x, h = self._row_parallel(ctx.view(rows, H * D), ly.o, x, ly.ln2)
      qc = self._skinny(h, ly.cq).view(rows, H, D)
      if self.cross_mma:
        decode_cross_attention_mma(qc, self.cross_k[i], self.cross_v[i], self.enc_mask_u8, ctx,
                                   self.k, self.enc_len)
        cc = ctx
      else:
        cc = attn_ops.flash_attention(qc.view(self.b, self.k, H, D),
                                      self.cross_k[i].transpose(1, 2),
                                      self.cross_v[i].transpose(1, 2), key_mask=self.enc_mask)
      x, h = self._row_parallel(cc.reshape(rows, H * D), ly.co, x, ly.ln3)
      g = native.gemm(h, ly.wi0, b2=ly.wi1)
      x, h = self._row_parallel(g, ly.wo, x, next_ln1)
    logits = native.gemm(h, self.w_logits, out_dtype=torch.float32, alpha=self.logit_scale)
    return logits if self.link is None else self.link.gather_logits(logits)

  def _row_parallel(self, a, w, residual, next_norm_scale):
    """(x, h): x = a @ w + residual and h = rmsnorm(x) * next_norm_scale, for a projection whose
    input features may be split over the model axis (the partial products are then summed
    over the ranks: one all-reduce site of the step)."""
    if self.link is not None:
      return self.link.all_reduce(a, w, residual, _splits(w.shape[0], w.shape[1], self.rows),
                                  norm_scale=next_norm_scale)
    if self.rows > 512:
      x = native.gemm(a, w, residual=residual)
      return x, native.rmsnorm_fwd(x, next_norm_scale, 1e-6)[0]
    if self.cluster_gemm:
      x = native.gemm_skinny(a, w, residual=residual)
      if x is not None:
        return x, native.rmsnorm_fwd(x, next_norm_scale, 1e-6)[0]
    return native.gemm_splitk_norm(a, w, _splits(w.shape[0], w.shape[1], self.rows),
                                   residual=residual, scale=next_norm_scale, eps=1e-6,
                                   workspace=self._workspace())

  def _skinny(self, a, w, residual=None):
    """a[rows, K] @ w[K, N] (+ residual) with K split over CTAs when rows are few."""
    if self.rows > 512:
      return native.gemm(a, w, residual=residual)
    if self.cluster_gemm:
      x = native.gemm_skinny(a, w, residual=residual)
      if x is not None:
        return x
    return native.gemm_splitk(a, w, _splits(w.shape[0], w.shape[1], self.rows),
                              residual=residual, workspace=self._workspace(),
                              workspace_is_clear=True)

  def _workspace(self) -> torch.Tensor:
    if self._ws is None:
      # zero once; every finishing kernel leaves what it read zero again
      self._ws = torch.zeros(self.rows * max(self.c.emb_dim, self.H * self.D),
                             dtype=torch.float32, device=self.dev)
    return self._ws

  def _beam_step(self, flat_logits: torch.Tensor) -> None:
    """One step of the search state update. Beam widths 1, 2, 4 and 8 run the two native
    kernels of csrc/beam.cu (log-softmax partials + candidate selection, then all of the
    bookkeeping per example); other widths run the same algorithm as tensor ops."""
    if self.k in (1, 2, 4, 8) and flat_logits.dtype == torch.float32:
      if self._beam_scratch is None:
        self._beam_scratch = native.BeamStepScratch(self.b, self.k, flat_logits.shape[1], self.dev)
      native.beam_step(flat_logits, batch=self.b, beams=self.k, eos_id=self.eos,
                       alpha=self.alpha, min_brevity=self.min_brevity, live_lp=self.live_lp,
                       live_seqs=self.live_seqs, fin_seqs=self.fin_seqs,
                       fin_scores=self.fin_scores, fin_flags=self.fin_flags, ancestry=self.anc,
                       cur=self.cur, terminated=self.terminated, scratch=self._beam_scratch)
      return
    self._beam_step_tensor_ops(flat_logits)

  def _beam_step_tensor_ops(self, flat_logits: torch.Tensor) -> None:
    b, k, L = self.b, self.k, self.L
    ci = self.cur.long()
    logits = flat_logits.view(b, k, -1)
    V = logits.shape[-1]
    log_probs = torch.log_softmax(logits, dim=-1) + self.live_lp[:, :, None]
    topk_lp, topk_idx = torch.topk(log_probs.view(b, k * V), 2 * k, dim=-1)
    topk_ids = topk_idx % V
    topk_beam = topk_idx // V
    nxt = (ci + 1).view(1, 1, 1)
    topk_seq = self.live_seqs.gather(1, topk_beam[:, :, None].expand(b, 2 * k, L))
    topk_seq = topk_seq.scatter(2, nxt.expand(b, 2 * k, 1), topk_ids[:, :, None])
    newly_finished = topk_ids == self.eos
    new_lp = topk_lp + newly_finished.float() * NEG_INF
    _, alive_idx = torch.topk(new_lp, k, dim=-1)
    alive_idx = torch.flip(alive_idx, dims=[1])  # ascending, like the reference
    parent = topk_beam.gather(1, alive_idx)
    self.live_seqs.copy_(topk_seq.gather(1, alive_idx[:, :, None].expand(b, k, L)))
    self.live_lp.copy_(new_lp.gather(1, alive_idx))
    # ancestry of the reselected beams: history of the parent, plus the parent's slot for the
    # position that was just written
    anc = self.anc.gather(1, parent[:, :, None].expand(b, k, L))
    anc = anc.scatter(2, ci.view(1, 1, 1).expand(b, k, 1), parent[:, :, None].to(torch.int32))
    self.anc.copy_(anc)
    # finished hypotheses
    length = (ci + 1).float()
    penalty = torch.pow((5.0 + length) / 6.0, self.alpha)
    new_scores = topk_lp / penalty + (~newly_finished).float() * NEG_INF
    all_seqs = torch.cat([self.fin_seqs, topk_seq], dim=1)
    all_scores = torch.cat([self.fin_scores, new_scores], dim=1)
    all_flags = torch.cat([self.fin_flags, newly_finished], dim=1)
    _, keep = torch.topk(all_scores, k, dim=-1)
    keep = torch.flip(keep, dims=[1])
    self.fin_seqs.copy_(all_seqs.gather(1, keep[:, :, None].expand(b, k, L)))
    self.fin_scores.copy_(all_scores.gather(1, keep))
    self.fin_flags.copy_(all_flags.gather(1, keep))
    self.cur.add_(1)
    # termination test for the NEXT step (t5x/decoding.py:1279-1312)
    best_live = self.live_lp[:, -1:] / self.min_brevity
    worst_fin = self.fin_scores.min(dim=1, keepdim=True).values
    worst_fin = torch.where(self.fin_flags, worst_fin.expand(b, k),
                            torch.full((b, k), NEG_INF, device=self.dev))
    self.terminated.copy_((worst_fin > best_live).all().view(1))

  def _step(self):
    if self.chain_level:
      with native.chained_launches(self.chain_level):
        self._beam_step(self._model_step())
    else:
      self._beam_step(self._model_step())

  # ------------------------------------------------------------------------------------------
  def decode(self, encoder_input_tokens: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """-> ([batch, beams, max_decode_len] sequences, [batch, beams] scores), ascending."""
    assert encoder_input_tokens.shape[0] == self.b
    with torch.no_grad():
      if self.graph is not None and encoder_input_tokens.shape[1] != self._graph_enc_len:
        self.graph = None  # the captured step has the encoder length in its arguments
      self._encode(encoder_input_tokens)
      self._reset()
      if self.use_graph and self.graph is None:
        # one eager step builds tensor maps and allocator pools, then the step is captured
        self._step()
        self._reset()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        n0 = native.launch_count()
        with torch.cuda.graph(g):
          self._step()
        self.kernels_per_step = native.launch_count() - n0
        self.graph = g
        self._graph_enc = (list(self.cross_k), list(self.cross_v), self.enc_mask,
                           self.enc_mask_u8)
        self._graph_enc_len = encoder_input_tokens.shape[1]
      elif self.use_graph:
        # the captured graph reads the encoder products through fixed buffers
        for dst, src in zip(self._graph_enc[0] + self._graph_enc[1], self.cross_k + self.cross_v):
          if dst is not src:
            dst.copy_(src)
        if self._graph_enc[2] is not self.enc_mask:
          self._graph_enc[2].copy_(self.enc_mask)
        self.cross_k, self.cross_v = list(self._graph_enc[0]), list(self._graph_enc[1])
        self.enc_mask = self._graph_enc[2]
        if self._graph_enc[3] is not self.enc_mask_u8:
          self._graph_enc[3].copy_(self.enc_mask_u8)
        self.enc_mask_u8 = self._graph_enc[3]
      max_steps = self.L - 1
      for step in range(max_steps):
        if step % self.check_period == 0 and step > 0 and bool(self.terminated.item()):
          break
        if self.graph is not None:
          self.graph.replay()
          self.replays += 1
        else:
          self._step()
      any_fin = self.fin_flags.any(dim=1)
      seqs = torch.where(any_fin[:, None, None], self.fin_seqs, self.live_seqs)
      scores = torch.where(any_fin[:, None], self.fin_scores, self.live_lp)
    return seqs[:, :, 1:].clone(), scores.clone()
