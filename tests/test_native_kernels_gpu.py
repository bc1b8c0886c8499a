"""Numerics of every sm_100a kernel against fp32 PyTorch statements of the same op."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def rel(a, b):
  a, b = a.float(), b.float()
  return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.fixture(scope="module")
def N():
  from t5x_b200.ops import native
  assert torch.cuda.is_available()
  native.lib()
  return native


BF16_TOL = 4e-3


@pytest.mark.parametrize("shape", [(128, 128, 64), (128, 256, 64), (256, 256, 128), (384, 512, 320),
                                   (304, 200, 136), (1000, 264, 72), (2048, 1280, 1024)])
@pytest.mark.parametrize("ta", [0, 1])
@pytest.mark.parametrize("tb", [0, 1])
def test_gemm_layouts(N, shape, ta, tb):
  M, Nn, K = shape
  torch.manual_seed(0)
  A = torch.randn(K, M, device="cuda").bfloat16().t() if ta else torch.randn(M, K, device="cuda").bfloat16()
  B = torch.randn(Nn, K, device="cuda").bfloat16().t() if tb else torch.randn(K, Nn, device="cuda").bfloat16()
  C = N.gemm(A, B)
  N.check_status()
  assert rel(C, A.float() @ B.float()) < BF16_TOL


@pytest.mark.parametrize("shape", [(256, 256, 64), (512, 768, 256), (384, 512, 320),
                                   (304, 200, 136), (1000, 264, 72), (2048, 1280, 1024),
                                   (4096, 4096, 512)])
@pytest.mark.parametrize("ta", [0, 1])
@pytest.mark.parametrize("tb", [0, 1])
def test_gemm_cta_pairs(N, shape, ta, tb):
  """The cta_group::2 kernel (forced on) against fp32 matmul, all operand layouts."""
  M, Nn, K = shape
  torch.manual_seed(0)
  A = torch.randn(K, M, device="cuda").bfloat16().t() if ta else torch.randn(M, K, device="cuda").bfloat16()
  B = torch.randn(Nn, K, device="cuda").bfloat16().t() if tb else torch.randn(K, Nn, device="cuda").bfloat16()
  N.gemm_set_pair_mode(2)
  try:
    C = N.gemm(A, B)
    N.check_status()
  finally:
    N.gemm_set_pair_mode(1)
  assert rel(C, A.float() @ B.float()) < BF16_TOL


def test_gemm_cta_pairs_epilogues(N):
  torch.manual_seed(1)
  M, Nn, K = 768, 640, 256
  A = torch.randn(M, K, device="cuda").bfloat16()
  B = (torch.randn(K, Nn, device="cuda") * 0.1).bfloat16()
  R = torch.randn(M, Nn, device="cuda").bfloat16()
  ref = A.float() @ B.float()
  N.gemm_set_pair_mode(2)
  try:
    assert rel(N.gemm(A, B, residual=R), ref + R.float()) < BF16_TOL
    Cf = torch.ones(M, Nn, device="cuda")
    N.gemm(A, B, out=Cf, accumulate=True)
    assert rel(Cf, ref + 1) < 1e-5
    W = (torch.randn(K, 2 * Nn, device="cuda") * 0.1).bfloat16()
    H = torch.empty(M, 2 * Nn, device="cuda", dtype=torch.bfloat16)
    G = N.gemm(A, W[:, :Nn], b2=W[:, Nn:], save_h=H)
    h = A.float() @ W.float()
    assert rel(G, torch.nn.functional.gelu(h[:, :Nn], approximate="tanh") * h[:, Nn:]) < BF16_TOL
    assert rel(H, h) < BF16_TOL
    Ab = torch.randn(3, 520, 128, device="cuda").bfloat16()
    Bb = torch.randn(3, 128, 264, device="cuda").bfloat16()
    assert rel(N.gemm(Ab, Bb), Ab.float() @ Bb.float()) < BF16_TOL
    N.check_status()
  finally:
    N.gemm_set_pair_mode(1)


def test_gemm_epilogues(N):
  torch.manual_seed(1)
  M, Nn, K = 512, 384, 256
  A = torch.randn(M, K, device="cuda").bfloat16()
  B = (torch.randn(K, Nn, device="cuda") * 0.1).bfloat16()
  R = torch.randn(M, Nn, device="cuda").bfloat16()
  ref = A.float() @ B.float()
  assert rel(N.gemm(A, B, residual=R), ref + R.float()) < BF16_TOL
  Cf = torch.ones(M, Nn, device="cuda")
  N.gemm(A, B, out=Cf, accumulate=True)
  assert rel(Cf, ref + 1) < 1e-5
  assert rel(N.gemm(A, B, out_dtype=torch.float32), ref) < 1e-5
  assert rel(N.gemm(A, B, out_dtype=torch.float32, alpha=0.5), 0.5 * ref) < 1e-5
  W = (torch.randn(K, 2 * Nn, device="cuda") * 0.1).bfloat16()
  H = torch.empty(M, 2 * Nn, device="cuda", dtype=torch.bfloat16)
  G = N.gemm(A, W[:, :Nn], b2=W[:, Nn:], save_h=H)
  h = A.float() @ W.float()
  assert rel(G, torch.nn.functional.gelu(h[:, :Nn], approximate="tanh") * h[:, Nn:]) < BF16_TOL
  assert rel(H, h) < BF16_TOL
  Ab = torch.randn(3, 200, 128, device="cuda").bfloat16()
  Bb = torch.randn(3, 128, 136, device="cuda").bfloat16()
  assert rel(N.gemm(Ab, Bb), Ab.float() @ Bb.float()) < BF16_TOL
  # strided output (a column slice of a wider matrix)
  wide = torch.zeros(M, 3 * Nn, device="cuda", dtype=torch.bfloat16)
  N.gemm(A, B, out=wide[:, Nn:2 * Nn])
  assert rel(wide[:, Nn:2 * Nn], ref) < BF16_TOL and float(wide[:, :Nn].abs().max()) == 0.0
  N.check_status()


def test_rmsnorm(N):
  torch.manual_seed(2)
  for T, d in [(1000, 4096), (77, 512), (33, 768), (5000, 768), (300, 1024), (64, 2048), (40, 8192)]:
    x = torch.randn(T, d, device="cuda").bfloat16()
    sc = torch.rand(d, device="cuda") + 0.5
    y, rstd = N.rmsnorm_fwd(x, sc, 1e-6)
    xf = x.float().requires_grad_(True)
    scp = sc.clone().requires_grad_(True)
    yr = xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + 1e-6) * scp
    assert rel(y, yr) < BF16_TOL
    dy = torch.randn(T, d, device="cuda").bfloat16()
    dres = torch.randn(T, d, device="cuda").bfloat16()
    yr.backward(dy.float())
    dsc = torch.zeros(d, device="cuda")
    dx = N.rmsnorm_bwd(dy, x, sc, rstd, dres, dsc)
    assert rel(dx, xf.grad + dres.float()) < BF16_TOL
    assert rel(dsc, scp.grad) < 1e-4


def test_gated_gelu(N):
  torch.manual_seed(3)
  T, dff = 300, 2048
  h = torch.randn(T, 2 * dff, device="cuda").bfloat16()
  dg = torch.randn(T, dff, device="cuda").bfloat16()
  hf = h.float().requires_grad_(True)
  g = torch.nn.functional.gelu(hf[:, :dff], approximate="tanh") * hf[:, dff:]
  g.backward(dg.float())
  assert rel(N.gated_gelu_fwd(h), g) < BF16_TOL
  hh, dgg = h.clone(), dg.clone()
  N.gated_gelu_bwd_(dgg, hh, True)
  assert rel(hh, hf.grad) < BF16_TOL and rel(dgg, g) < BF16_TOL


def test_embedding(N):
  torch.manual_seed(4)
  V, d = 5000, 512
  tab = torch.randn(V, d, device="cuda").bfloat16()
  ids = torch.randint(0, V, (7, 33), device="cuda")
  assert rel(N.embedding_fwd(ids, tab), tab[ids]) == 0.0
  dt = torch.zeros(V, d, device="cuda")
  do = torch.randn(7, 33, d, device="cuda").bfloat16()
  N.embedding_bwd_(ids, do, dt)
  ref = torch.zeros(V, d, device="cuda").index_add_(0, ids.view(-1), do.view(-1, d).float())
  assert rel(dt, ref) < 1e-6
  # vocab-parallel slice: ids outside [start, start+rows) give zeros
  part = N.embedding_fwd(ids, tab[1000:3000].contiguous(), vocab_start=1000)
  own = ((ids >= 1000) & (ids < 3000))[..., None]
  assert rel(part, tab[ids] * own) == 0.0


def test_cross_entropy(N):
  torch.manual_seed(5)
  T, V = 300, 32128
  lg = torch.randn(T, V, device="cuda") * 3
  tg = torch.randint(0, V, (T,), device="cuda")
  st, av, ai = N.ce_stats(lg, tg)
  lse = st[:, 0] + torch.log(st[:, 1])
  assert rel(lse, torch.logsumexp(lg, -1)) < 1e-6
  assert rel(st[:, 2], lg.gather(1, tg[:, None]).squeeze()) == 0.0
  assert bool((ai.long() == lg.argmax(-1)).all())
  rs = torch.rand(T, device="cuda")
  dl = N.ce_grad(lg, tg, lse, rs, 1e-4, 1.0, 0.0)
  lgr = lg.clone().requires_grad_(True)
  l2 = torch.logsumexp(lgr, -1)
  ((l2 - lgr.gather(1, tg[:, None]).squeeze() + 1e-4 * l2 * l2) * rs).sum().backward()
  assert rel(dl, lgr.grad) < BF16_TOL


@pytest.mark.parametrize("shape", [(512, 1024, 1), (1024, 512, 0), (300, 260, 1), (130, 32128, 1)])
def test_adafactor_factored(N, shape):
  R, C, norm = shape
  torch.manual_seed(6)
  p = torch.randn(R, C, device="cuda") * 0.05
  g = torch.randn(R, C, device="cuda") * 0.01
  vr = torch.rand(R, device="cuda") * 1e-4
  vc = torch.rand(C, device="cuda") * 1e-4
  pb = torch.empty(R, C, device="cuda", dtype=torch.bfloat16)
  scratch = torch.empty(N.adafactor_scratch_floats(1, R, C), device="cuda")
  decay, lr = 0.8, 0.01
  p0, vr0, vc0 = p.clone(), vr.clone(), vc.clone()
  N.adafactor_factored_(p, g, vr, vc, None, pb, scratch, batch=1, rows=R, cols=C,
                        row_is_normalized=norm, lr=lr, decay=decay, eps1=1e-30, eps2=1e-3,
                        clip_threshold=1.0, weight_decay=0.0, beta1=0.0, max_param_scale=0.0,
                        flags=N.AF_PARAM_SCALE | N.AF_CLIP, ld_bf16=C)
  gs = g * g + 1e-30
  nvr = decay * vr0 + (1 - decay) * gs.mean(1)
  nvc = decay * vc0 + (1 - decay) * gs.mean(0)
  if norm:
    rf, cf = (nvr / nvr.mean()) ** -0.5, nvc ** -0.5
  else:
    rf, cf = nvr ** -0.5, (nvc / nvc.mean()) ** -0.5
  u = g * rf[:, None] * cf[None, :]
  u = u / torch.clamp(u.pow(2).mean().sqrt(), min=1.0)
  pn = p0 - lr * torch.clamp(p0.pow(2).mean().sqrt(), min=1e-3) * u
  assert rel(p, pn) < 1e-5 and rel(vr, nvr) < 1e-5 and rel(vc, nvc) < 1e-5
  assert rel(pb, pn) < BF16_TOL
  N.check_status()


def test_adafactor_unfactored(N):
  torch.manual_seed(7)
  n = 5000
  p = torch.randn(1, n, device="cuda")
  g = torch.randn(1, n, device="cuda") * 0.1
  v = torch.rand(1, n, device="cuda") * 1e-3
  p0, v0 = p.clone(), v.clone()
  scratch = torch.empty(8, device="cuda")
  N.adafactor_unfactored_(p, g, v, None, None, scratch, batch=1, rows=1, cols=n, lr=0.01,
                          decay=0.8, eps1=1e-30, eps2=1e-3, clip_threshold=1.0, weight_decay=0.0,
                          beta1=0.0, max_param_scale=0.0, flags=N.AF_PARAM_SCALE | N.AF_CLIP)
  nv = 0.8 * v0 + 0.2 * (g * g + 1e-30)
  u = g * nv ** -0.5
  u = u / torch.clamp(u.pow(2).mean().sqrt(), min=1.0)
  pn = p0 - 0.01 * torch.clamp(p0.pow(2).mean().sqrt(), min=1e-3) * u
  assert rel(p, pn) < 1e-5 and rel(v, nv) < 1e-5


@pytest.mark.parametrize("shape", [(768, 768, 16384), (768, 2048, 8192), (320, 200, 12288)])
def test_weight_gradient_split_k(N, shape):
  """dW (+)= x^T dy with K cut into slices that add into the fp32 output atomically."""
  M, Nn, K = shape
  torch.manual_seed(0)
  x = torch.randn(K, M, device="cuda").to(torch.bfloat16)       # activations [tokens, in]
  dy = torch.randn(K, Nn, device="cuda").to(torch.bfloat16)     # [tokens, out]
  splits = N.wgrad_splits(M, Nn, K)
  assert splits > 1
  want = x.float().t() @ dy.float()
  out = torch.full((M, Nn), 7.0, device="cuda")
  N.gemm_splitk_accumulate(x.t(), dy, out, splits, accumulate=False)
  assert rel(out, want) < BF16_TOL
  N.gemm_splitk_accumulate(x.t(), dy, out, splits, accumulate=True)
  assert rel(out, 2 * want) < BF16_TOL
  # large outputs keep the single-pass kernel
  assert N.wgrad_splits(4096, 4096, 8192) == 1
  N.check_status()


@pytest.mark.parametrize("rows,vocab,tied,smoothing,scale", [
    (300, 32128, False, 0.0, 1.0), (1824, 32128, False, 0.1, 1.0), (77, 1000, True, 0.0, 0.125),
    (513, 4096, False, 0.05, 1.0)])
def test_projection_fused_with_cross_entropy(N, rows, vocab, tied, smoothing, scale):
  """`logits_cross_entropy` keeps no logits: forward partials come out of the GEMM epilogue and
  backward recomputes the tiles. Checked against fp32 autograd over materialised logits, and
  against the materialised-logits kernels of the same library."""
  import os
  from t5x_b200.ops import functional as F, reference as ref
  torch.manual_seed(rows + vocab)
  d = 256
  h = (torch.randn(rows, d, device="cuda") * 0.7).bfloat16().requires_grad_(True)
  w32 = torch.randn(vocab, d, device="cuda") * 0.2 if tied else torch.randn(d, vocab, device="cuda") * 0.2
  w = w32.clone().requires_grad_(True)
  w.bf16 = w32.bfloat16()
  tg = torch.randint(0, vocab, (rows,), device="cuda")
  wt = torch.rand(rows, device="cuda")
  z_loss = 1e-4

  def run(fused):
    os.environ["T5X_B200_FUSED_CE"] = "1" if fused else "0"
    h.grad = w.grad = None
    loss, z, correct = F.logits_cross_entropy(h, w, tg, z_loss=z_loss, label_smoothing=smoothing,
                                              logits_scale=scale)
    (loss * wt).sum().backward()
    return loss.detach(), z.detach(), correct, h.grad.clone(), w.grad.clone()

  try:
    n0 = N.launch_count()
    got = run(True)
    assert N.launch_count() > n0
    old = run(False)
  finally:
    os.environ.pop("T5X_B200_FUSED_CE", None)
  N.check_status()
  hr = h.detach().float().requires_grad_(True)
  wr = w.bf16.float().requires_grad_(True)
  logits = (hr @ (wr.t() if tied else wr)) * scale
  rl, rz, _, ram = ref.token_cross_entropy(logits, tg, z_loss, smoothing)
  (rl * wt).sum().backward()
  assert rel(got[0], rl) < 2e-5 and rel(got[1], rz) < 1e-4
  agree = (got[2] == (ram == tg)).float().mean()
  assert float(agree) > 0.995  # arg-max ties between near-equal logits may differ
  assert rel(got[3], hr.grad) < BF16_TOL
  assert rel(got[4], wr.grad) < BF16_TOL
  # and the two library paths agree with each other more tightly than with fp32
  assert rel(got[0], old[0]) < 1e-5
  assert rel(got[3], old[3]) < 6e-3 and rel(got[4], old[4]) < 6e-3


def test_fused_adamw_matches_the_generic_chain():
  """clip_by_global_norm -> adamw through the one-kernel path against the same chain evaluated
  transformation by transformation with tensor ops (fp32 throughout), three steps."""
  from t5x_b200 import optimizers
  from t5x_b200.ops import native

  def run(fused):
    torch.manual_seed(5)
    params = {"a": {"kernel": torch.randn(384, 515, device="cuda")},
              "b": {"scale": torch.randn(1027, device="cuda")}}
    for leaf in (params["a"]["kernel"], params["b"]["scale"]):
      leaf.bf16 = leaf.to(torch.bfloat16)
    opt_def = optimizers.chain([optimizers.clip_by_global_norm(0.5),
                                optimizers._adamw(3e-3, weight_decay=0.05)])
    assert opt_def.fused_plan is not None
    if not fused:
      opt_def.fused_plan = None
    opt = opt_def.create(params)
    for step in range(3):
      g = {"a": {"kernel": torch.randn(384, 515, device="cuda") * (step + 1)},
           "b": {"scale": torch.randn(1027, device="cuda")}}
      opt = opt.apply_gradient(g)
    native.check_status()
    adam = opt.state.param_states["1"]["0"]
    return opt.target, adam

  (pf, sf), (pg, sg) = run(True), run(False)
  for path in (("a", "kernel"), ("b", "scale")):
    f, g = pf[path[0]][path[1]], pg[path[0]][path[1]]
    torch.testing.assert_close(f, g, rtol=2e-5, atol=2e-6)
    torch.testing.assert_close(f.bf16.float(), f, rtol=8e-3, atol=1e-3)
    for slot in ("mu", "nu"):
      torch.testing.assert_close(sf[slot][path[0]][path[1]], sg[slot][path[0]][path[1]],
                                 rtol=2e-5, atol=1e-7)
  assert int(sf["count"]) == int(sg["count"]) == 3


@pytest.mark.parametrize("options", [
    dict(beta1=0.9),
    dict(weight_decay_rate=0.01, multiply_by_parameter_scale=False),
    dict(beta1=0.9, weight_decay_rate=0.02, max_parameter_scale=0.04),
    dict(factored=False, beta1=0.5),
    dict(skip_nan_updates=True),
    dict(global_norm_clip_threshold=0.05),
])
def test_adafactor_options_on_gpu_match_the_cpu_statement(options):
  """The optimizer with momentum, weight decay, a parameter-scale ceiling, NaN skipping and
  global-norm clipping: three steps through the native kernels against the same class on CPU
  tensors (plain tensor ops)."""
  from t5x_b200 import adafactor
  torch.manual_seed(11)
  shapes = {"dense": {"kernel": (256, 384)}, "norm": {"scale": (384,)},
            "embed": {"table": (130, 256)}}
  init = {k: {n: torch.randn(s) * 0.05 for n, s in v.items()} for k, v in shapes.items()}
  grads = [{k: {n: torch.randn(s) * 0.02 for n, s in v.items()} for k, v in shapes.items()}
           for _ in range(3)]
  if options.get("skip_nan_updates"):
    grads[1]["dense"]["kernel"][3, 7] = float("nan")

  def run(device):
    params = {k: {n: t.clone().to(device) for n, t in v.items()} for k, v in init.items()}
    opt = adafactor.Adafactor(decay_rate=0.8, step_offset=0, **options).create(params)
    for g in grads:
      g_dev = {k: {n: t.clone().to(device) for n, t in v.items()} for k, v in g.items()}
      opt = opt.apply_gradient(g_dev, learning_rate=0.01)
    return opt

  cpu, gpu = run("cpu"), run("cuda")
  from t5x_b200.ops import native
  native.check_status()
  for k, v in shapes.items():
    for n in v:
      a, b = gpu.target[k][n].float().cpu(), cpu.target[k][n].float()
      if options.get("skip_nan_updates"):
        assert not torch.isnan(a).any()
      assert rel(a, b) < 2e-5, (k, n, rel(a, b))
      for slot, val in cpu.state.param_states[k][n].items():
        got = gpu.state.param_states[k][n][slot].float().cpu()
        if val.numel() > 1:
          assert rel(got, val.float()) < 2e-5, (k, n, slot)
