"""T5 layer helpers on the CPU: attention / causal / decoder masks (unpacked, packed,
prefix-LM, composite causal attention), mask and bias combination, the dense attention
function, projections, embeddings and relative position biases (the behaviours of
t5x/examples/t5/layers_test.py; the bucket function is checked against the independent
implementation in the `transformers` package when that is importable)."""
import numpy as np
import pytest
import torch

from t5x_b200.models.t5 import layers
from t5x_b200.ops import reference as ref


def test_make_attention_mask_multiply_and_equal():
  tokens = torch.tensor([[7, 0, 0], [8, 5, 0]])
  mask = layers.make_attention_mask(tokens > 0, tokens > 0, dtype=torch.int32)
  assert mask.shape == (2, 1, 3, 3)
  assert mask[0, 0].tolist() == [[1, 0, 0], [0, 0, 0], [0, 0, 0]]
  assert mask[1, 0].tolist() == [[1, 1, 0], [1, 1, 0], [0, 0, 0]]
  seg = torch.tensor([[1, 1, 2, 2, 2, 0], [1, 1, 1, 2, 0, 0]])
  mask = layers.make_attention_mask(seg, seg, pairwise_fn=torch.eq, dtype=torch.int32)
  assert mask.shape == (2, 1, 6, 6)
  # padding is not special here: equal ids (also 0 == 0) attend
  assert mask[0, 0].tolist() == [[1, 1, 0, 0, 0, 0], [1, 1, 0, 0, 0, 0], [0, 0, 1, 1, 1, 0],
                                 [0, 0, 1, 1, 1, 0], [0, 0, 1, 1, 1, 0], [0, 0, 0, 0, 0, 1]]
  assert mask[1, 0, 4].tolist() == [0, 0, 0, 0, 1, 1]


def test_make_causal_mask():
  y = layers.make_causal_mask(torch.tensor([[7, 0, 0], [8, 5, 0]]))
  assert y.shape == (2, 1, 3, 3)
  tri = [[1.0, 0.0, 0.0], [1.0, 1.0, 0.0], [1.0, 1.0, 1.0]]
  assert y[0, 0].tolist() == tri and y[1, 0].tolist() == tri   # padding plays no part


def test_combine_masks_and_biases():
  masks = [torch.tensor([0., 1, 0, 1]), None, torch.tensor([1., 1, 1, 1]), torch.tensor([1., 1, 1, 0])]
  assert layers.combine_masks(*masks).tolist() == [0, 1, 0, 0]
  assert layers.combine_masks(None, None) is None
  biases = [torch.tensor([0., 1, 0, 1]), None, torch.tensor([0., 1, 1, 1]), torch.tensor([0., 1, 1, 0])]
  assert layers.combine_biases(*biases).tolist() == [0, 3, 2, 2]
  assert layers.combine_biases(None) is None


def test_decoder_mask_language_model():
  mask = layers.make_decoder_mask(torch.tensor([6, 7, 3, 0]))
  assert mask.tolist() == [[[1, 0, 0, 0], [1, 1, 0, 0], [1, 1, 1, 0], [0, 0, 0, 0]]]
  packed = layers.make_decoder_mask(torch.tensor([[6, 7, 3, 4, 5, 0]]),
                                    decoder_segment_ids=torch.tensor([[1, 1, 1, 2, 2, 0]]))
  assert packed[0, 0].tolist() == [[1, 0, 0, 0, 0, 0], [1, 1, 0, 0, 0, 0], [1, 1, 1, 0, 0, 0],
                                   [0, 0, 0, 1, 0, 0], [0, 0, 0, 1, 1, 0], [0, 0, 0, 0, 0, 0]]


def test_decoder_mask_prefix_lm():
  mask = layers.make_decoder_mask(torch.tensor([[5, 6, 7, 3, 4, 0]]),
                                  decoder_causal_attention=torch.tensor([[1, 1, 1, 0, 0, 0]]))
  assert mask[0, 0].tolist() == [[1, 1, 1, 0, 0, 0], [1, 1, 1, 0, 0, 0], [1, 1, 1, 0, 0, 0],
                                 [1, 1, 1, 1, 0, 0], [1, 1, 1, 1, 1, 0], [0, 0, 0, 0, 0, 0]]
  packed = layers.make_decoder_mask(
      torch.tensor([[5, 6, 7, 8, 3, 4, 0]]),
      decoder_causal_attention=torch.tensor([[1, 1, 0, 1, 1, 0, 0]]),
      decoder_segment_ids=torch.tensor([[1, 1, 1, 2, 2, 2, 0]]))
  assert packed[0, 0].tolist() == [
      [1, 1, 0, 0, 0, 0, 0], [1, 1, 0, 0, 0, 0, 0], [1, 1, 1, 0, 0, 0, 0], [0, 0, 0, 1, 1, 0, 0],
      [0, 0, 0, 1, 1, 0, 0], [0, 0, 0, 1, 1, 1, 0], [0, 0, 0, 0, 0, 0, 0]]
  two = layers.make_decoder_mask(torch.tensor([[6, 7, 3, 0], [4, 5, 0, 0]]),
                                 decoder_causal_attention=torch.tensor([[1, 1, 0, 0], [1, 0, 0, 0]]))
  assert two.shape == (2, 1, 4, 4)
  assert two[0, 0].tolist() == [[1, 1, 0, 0], [1, 1, 0, 0], [1, 1, 1, 0], [0, 0, 0, 0]]
  assert two[1, 0].tolist() == [[1, 0, 0, 0], [1, 1, 0, 0], [0, 0, 0, 0], [0, 0, 0, 0]]


def test_decoder_mask_composite_causal_attention():
  """Several fully visible spans in one sequence: their positions all see each other."""
  mask = layers.make_decoder_mask(torch.tensor([[6, 7, 3, 4, 8, 9, 0]]),
                                  decoder_causal_attention=torch.tensor([[1, 1, 0, 0, 1, 1, 0]]))
  assert mask[0, 0].tolist() == [
      [1, 1, 0, 0, 1, 1, 0], [1, 1, 0, 0, 1, 1, 0], [1, 1, 1, 0, 0, 0, 0], [1, 1, 1, 1, 0, 0, 0],
      [1, 1, 1, 1, 1, 1, 0], [1, 1, 1, 1, 1, 1, 0], [0, 0, 0, 0, 0, 0, 0]]
  packed = layers.make_decoder_mask(
      torch.tensor([[6, 7, 3, 4, 8, 9, 2, 3, 4]]),
      decoder_causal_attention=torch.tensor([[1, 1, 0, 0, 1, 1, 1, 1, 0]]),
      decoder_segment_ids=torch.tensor([[1, 1, 1, 1, 1, 1, 2, 2, 2]]))
  assert packed[0, 0, 5].tolist() == [1, 1, 1, 1, 1, 1, 0, 0, 0]
  assert packed[0, 0, 6].tolist() == [0, 0, 0, 0, 0, 0, 1, 1, 0]
  assert packed[0, 0, 8].tolist() == [0, 0, 0, 0, 0, 0, 1, 1, 1]


def test_dot_product_attention_against_a_manual_softmax():
  torch.manual_seed(0)
  b, q, k, h, d = 2, 3, 5, 4, 8
  query, key, value = torch.randn(b, q, h, d), torch.randn(b, k, h, d), torch.randn(b, k, h, d)
  bias = torch.randn(b, h, q, k)
  out = layers.dot_product_attention(query, key, value, bias=bias)
  assert out.shape == (b, q, h, d)
  logits = torch.einsum("bqhd,bkhd->bhqk", query, key) + bias   # no 1/sqrt(d): T5 folds it in
  want = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(logits, -1), value)
  torch.testing.assert_close(out, want)
  # a -1e10 bias removes a key
  bias2 = torch.zeros(b, h, q, k)
  bias2[..., -1] = -1e10
  out2 = layers.dot_product_attention(query, key, value, bias=bias2)
  want2 = layers.dot_product_attention(query, key[:, :-1], value[:, :-1])
  torch.testing.assert_close(out2, want2)


def test_dense_general_and_mlp_block_shapes_and_axes():
  dense = layers.DenseGeneral(6, 10, kernel_axes=("embed", "mlp"))
  assert tuple(dense.kernel.shape) == (6, 10) and tuple(dense.kernel.axes) == ("embed", "mlp")
  x = torch.randn(2, 3, 6)
  torch.testing.assert_close(dense(x), x @ dense.kernel)
  assert not any(n.endswith("bias") for n, _ in dense.named_parameters())
  mlp = layers.MlpBlock(emb_dim=6, intermediate_dim=12, activations=("gelu", "linear"),
                        intermediate_dropout_rate=0.0)
  names = sorted(n for n, _ in mlp.named_parameters())
  assert names == ["wi_0.kernel", "wi_1.kernel", "wo.kernel"]
  y = mlp(x)
  assert y.shape == x.shape
  want = (ref.gelu_tanh(x @ mlp.wi_0.kernel) * (x @ mlp.wi_1.kernel)) @ mlp.wo.kernel
  torch.testing.assert_close(y, want, rtol=1e-5, atol=1e-5)
  single = layers.MlpBlock(emb_dim=6, intermediate_dim=12, activations=("relu",),
                           intermediate_dropout_rate=0.0)
  assert sorted(n for n, _ in single.named_parameters()) == ["wi.kernel", "wo.kernel"]
  torch.testing.assert_close(single(x), torch.relu(x @ single.wi.kernel) @ single.wo.kernel,
                             rtol=1e-5, atol=1e-5)


def test_embed_lookup_and_attend():
  emb = layers.Embed(num_embeddings=10, features=4)
  assert tuple(emb.embedding.shape) == (10, 4) and tuple(emb.embedding.axes) == ("vocab", "embed")
  ids = torch.tensor([[1, 9, 0], [3, 3, 2]])
  out = emb(ids)
  assert out.shape == (2, 3, 4)
  torch.testing.assert_close(out[1, 0], emb.embedding[3].detach())
  q = torch.randn(2, 3, 4)
  logits = emb.attend(q)
  assert logits.shape == (2, 3, 10)
  torch.testing.assert_close(logits, q @ emb.embedding.detach().t())


def test_relative_position_biases_shapes_and_sharing():
  rel = layers.RelativePositionBiases(num_buckets=12, max_distance=10, num_heads=3)
  assert tuple(rel.rel_embedding.shape) == (3, 12)
  assert tuple(rel.rel_embedding.axes) == ("heads", "relpos_buckets")
  for bidirectional in (True, False):
    out = rel(5, 7, bidirectional=bidirectional)
    assert out.shape == (1, 3, 5, 7)
    # the bias depends on key position minus query position only
    torch.testing.assert_close(out[0, :, 0, 1], out[0, :, 3, 4])
    torch.testing.assert_close(out[0, :, 2, 0], out[0, :, 4, 2])
  uni = rel(5, 7, bidirectional=False)
  # looking ahead is one bucket in the unidirectional scheme
  torch.testing.assert_close(uni[0, :, 0, 3], uni[0, :, 0, 6])
  bi = rel(5, 7, bidirectional=True)
  assert not torch.allclose(bi[0, :, 0, 1], bi[0, :, 0, 6])


@pytest.mark.parametrize("bidirectional", [True, False])
@pytest.mark.parametrize("num_buckets,max_distance", [(32, 128), (12, 10), (8, 64)])
def test_relative_position_bucket_against_an_independent_implementation(bidirectional, num_buckets,
                                                                         max_distance):
  modeling = pytest.importorskip("transformers.models.t5.modeling_t5")
  rel = torch.arange(-300, 301)[None, :].repeat(2, 1)
  want = modeling.T5Attention._relative_position_bucket(
      rel, bidirectional=bidirectional, num_buckets=num_buckets, max_distance=max_distance)
  got = ref.relative_position_bucket(rel, bidirectional, num_buckets, max_distance)
  assert got.tolist() == want.tolist()
  assert int(got.min()) >= 0 and int(got.max()) < num_buckets
