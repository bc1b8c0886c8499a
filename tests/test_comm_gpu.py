"""NVLink peer-memory kernels and the data-axis optimizer sharding built on them.

Multi-rank cases run as child processes (one per GPU) and need at least two GPUs; the
barrier-timeout case needs one: it waits on a flag that nothing sets and checks that the wait
gives up with a status instead of hanging."""
import json
import os
import signal
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
RANKS_TIMEOUT_S = 240


def _run_ranks(case, tmp_path, n=2, env=None):
  out = tmp_path / case
  out.mkdir(parents=True, exist_ok=True)
  e = dict(os.environ)
  e.update({"NCCL_NVLS_ENABLE": "0", "MASTER_ADDR": "127.0.0.1"})
  e.update(env or {})
  cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
         "--master-addr", "127.0.0.1", "--master-port", str(29500 + os.getpid() % 1000),
         os.path.join(HERE, "multi_gpu_worker.py"), case, str(out)]
  # own process group, so that a run that exceeds the limit is ended as a whole (the ranks are
  # grandchildren of this process)
  proc = subprocess.Popen(cmd, env=e, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True,
                          start_new_session=True)
  try:
    stdout, stderr = proc.communicate(timeout=RANKS_TIMEOUT_S)
  except subprocess.TimeoutExpired:
    os.killpg(proc.pid, signal.SIGKILL)
    stdout, stderr = proc.communicate()
    raise AssertionError(f"case {case!r} did not finish in {RANKS_TIMEOUT_S} s\n" +
                         stdout[-2000:] + stderr[-2000:])
  assert proc.returncode == 0, stdout[-3000:] + stderr[-3000:]
  return [json.load(open(out / f"rank{i}.json")) for i in range(n)]


def _need_two():
  if torch.cuda.device_count() < 2:
    pytest.skip("needs 2 GPUs")


def test_peer_reduce_push_barrier(tmp_path):
  _need_two()
  for res in _run_ranks("collectives", tmp_path):
    assert res["err_reduce"] < 1e-5
    assert res["ok_push"]


def test_sharded_optimizer_matches_all_reduce(tmp_path):
  _need_two()
  sharded = _run_ranks("train", tmp_path / "z")
  plain = _run_ranks("train", tmp_path / "p", env={"T5X_B200_OPTIMIZER_SHARDING": "0"})
  assert all(r["sharded"] for r in sharded) and not any(r["sharded"] for r in plain)
  # the layers' updates ran during the backward pass of the last microbatch
  assert all(r["overlapped"] > 0 for r in sharded)
  # replicas agree with each other, and the two gradient-reduction routes agree
  for run in (sharded, plain):
    assert abs(run[0]["param_sum"] - run[1]["param_sum"]) <= 1e-6 * run[0]["param_abs"]
    assert run[0]["loss"] == pytest.approx(run[1]["loss"], rel=1e-6)
    assert run[0]["slot_abs"] == pytest.approx(run[1]["slot_abs"], rel=1e-6)
  a, b = sharded[0], plain[0]
  assert a["loss"] == pytest.approx(b["loss"], rel=2e-3)
  assert a["param_abs"] == pytest.approx(b["param_abs"], rel=1e-4)
  assert a["bf16_abs"] == pytest.approx(a["param_abs"], rel=5e-3)
  for x, y in zip(a["first"], b["first"]):
    assert x == pytest.approx(y, rel=1e-2, abs=1e-4)


def test_sharded_weights_match_replicated_weights(tmp_path):
  """bf16 working weights of the transformer layers kept on their owners only and gathered
  layer by layer (T5X_B200_ZERO_SHARD_WEIGHTS=1) train exactly like replicated weights: the
  same kernels see the same operands."""
  _need_two()
  sharded = _run_ranks("train", tmp_path / "w", env={"T5X_B200_ZERO_SHARD_WEIGHTS": "1"})
  plain = _run_ranks("train", tmp_path / "p")
  assert all(r["weights_sharded"] for r in sharded) and not any(r["weights_sharded"] for r in plain)
  # the persistent weight buffer shrinks: replicated part + this rank's share of the layers
  assert sharded[0]["weight_elems"][0] < 0.8 * sharded[0]["weight_elems"][1]
  assert plain[0]["weight_elems"][0] == plain[0]["weight_elems"][1]
  assert sharded[0]["overlapped"] > 0
  for a, b in zip(sharded, plain):
    assert a["loss"] == pytest.approx(b["loss"], rel=1e-5)
    assert a["param_abs"] == pytest.approx(b["param_abs"], rel=1e-6)
    assert a["bf16_abs"] == pytest.approx(b["bf16_abs"], rel=1e-6)
    assert a["slot_abs"] == pytest.approx(b["slot_abs"], rel=1e-5)
    for x, y in zip(a["first"], b["first"]):
      assert x == pytest.approx(y, rel=1e-4, abs=1e-6)


def test_weight_metrics_under_the_sharded_optimizer(tmp_path):
  """Weight / gradient / update norms keep the optimizer sharded: each rank reports the
  parameters it owns and the ranks add up; the figures match the all-reduce run."""
  _need_two()
  env = {"T5X_TEST_WEIGHT_METRICS": "1"}
  sharded = _run_ranks("train", tmp_path / "z", env=env)
  plain = _run_ranks("train", tmp_path / "p", env={**env, "T5X_B200_OPTIMIZER_SHARDING": "0"})
  assert all(r["sharded"] for r in sharded) and not any(r["sharded"] for r in plain)
  assert len(sharded[0]["weight_metrics"]) >= 5
  for r in sharded[1:]:
    assert r["weight_metrics"] == pytest.approx(sharded[0]["weight_metrics"], rel=1e-6)
  for k, v in plain[0]["weight_metrics"].items():
    assert sharded[0]["weight_metrics"][k] == pytest.approx(v, rel=2e-3), k


@pytest.mark.parametrize("kind", ["adamw_clip", "adafactor_clip"])
def test_sharded_adamw_and_global_norm_clip_match_all_reduce(tmp_path, kind):
  """Optimizers whose update needs the norm of the whole gradient: owners reduce first, the
  squared norms are summed over the data axis, and the fused AdamW kernel (or Adafactor's own
  kernels) then update and push. Optimizer slots agree between ranks after `sync_replicas`."""
  _need_two()
  env = {"T5X_TEST_OPTIMIZER": kind}
  sharded = _run_ranks("train", tmp_path / "z", env=env)
  plain = _run_ranks("train", tmp_path / "p", env={**env, "T5X_B200_OPTIMIZER_SHARDING": "0"})
  assert all(r["sharded"] for r in sharded) and not any(r["sharded"] for r in plain)
  for run in (sharded, plain):
    assert abs(run[0]["param_sum"] - run[1]["param_sum"]) <= 1e-6 * run[0]["param_abs"]
    assert run[0]["slot_abs"] == pytest.approx(run[1]["slot_abs"], rel=1e-6)
  a, b = sharded[0], plain[0]
  assert a["loss"] == pytest.approx(b["loss"], rel=2e-3)
  assert a["param_abs"] == pytest.approx(b["param_abs"], rel=1e-4)
  assert a["slot_abs"] == pytest.approx(b["slot_abs"], rel=1e-2)
  assert a["bf16_abs"] == pytest.approx(a["param_abs"], rel=5e-3)
  for x, y in zip(a["first"], b["first"]):
    assert x == pytest.approx(y, rel=1e-2, abs=1e-4)


def test_sharded_optimizer_through_the_switch_matches_peer_loads(tmp_path):
  """The same three steps with the gradient sum taken by the NVSwitch (`multimem.ld_reduce`)
  and the weights pushed by one multicast store, against the peer-load form. Skipped where the
  fabric offers no multicast."""
  _need_two()
  switch = _run_ranks("train", tmp_path / "s", env={"T5X_B200_NVLS": "1"})
  if not all(r["nvls"] for r in switch):
    pytest.skip("no NVSwitch multicast on this box")
  plain = _run_ranks("train", tmp_path / "p")
  assert not any(r["nvls"] for r in plain)
  assert abs(switch[0]["param_sum"] - switch[1]["param_sum"]) <= 1e-6 * switch[0]["param_abs"]
  a, b = switch[0], plain[0]
  assert a["loss"] == pytest.approx(b["loss"], rel=2e-3)
  assert a["param_abs"] == pytest.approx(b["param_abs"], rel=1e-4)
  assert a["bf16_abs"] == pytest.approx(a["param_abs"], rel=5e-3)
  for x, y in zip(a["first"], b["first"]):
    assert x == pytest.approx(y, rel=1e-2, abs=1e-4)


def test_data_axis_selfcheck_passes(tmp_path):
  """`selfcheck.run` raises when an error exceeds its tolerance; here it must not."""
  _need_two()
  for res in _run_ranks("selfcheck", tmp_path):
    assert res["peer_reduce"] < 1e-5
    assert res["sharded_adafactor_vs_allreduce"] < 2e-2


def test_barrier_gives_up_when_a_peer_never_arrives():
  from t5x_b200.ops import comm, native
  pad = torch.zeros(256, dtype=torch.int32, device="cuda")
  # "two ranks" whose pads are both this buffer: rank 0 signals slot 0 and waits for slot 1,
  # which nobody writes.
  comm.barrier([pad.data_ptr(), pad.data_ptr()], rank=0, world=2, channel=0, epoch=1,
               spin_limit=2000)
  with pytest.raises(native.KernelStatusError, match="peer"):
    native.check_status()
  assert int(pad[0]) == 1 and int(pad[1]) == 0
  # the context is still usable and the status is cleared
  assert float(torch.ones(4, device="cuda").sum()) == 4.0
  native.check_status()


def test_moe_fused_exchange_matches_all_to_all(tmp_path):
  _need_two()
  fused = _run_ranks("moe", tmp_path / "f")
  plain = _run_ranks("moe", tmp_path / "p", env={"T5X_B200_MOE_FUSED": "0"})
  for a, b in zip(fused, plain):
    assert a["loss"] == pytest.approx(b["loss"], rel=2e-3)
    for key in ("wi", "wo", "router", "dense"):
      assert a[key] == pytest.approx(b[key], rel=2e-2), key
    for x, y in zip(a["wi_first"], b["wi_first"]):
      assert x == pytest.approx(y, rel=5e-2, abs=1e-3)


def test_fused_tensor_parallel_gemms(tmp_path):
  _need_two()
  for res in _run_ranks("tp_ops", tmp_path):
    for name, errs in res.items():
      for what, e in errs.items():
        assert e < 3e-2, (name, what, e)


def test_fused_tensor_parallel_training_matches_all_reduce(tmp_path):
  _need_two()
  fused = _run_ranks("tp_train", tmp_path / "f")
  plain = _run_ranks("tp_train", tmp_path / "p", env={"T5X_B200_TP_FUSED": "0"})
  assert all(r["fused"] for r in fused) and not any(r["fused"] for r in plain)
  a, b = fused[0], plain[0]
  assert fused[0]["loss"] == pytest.approx(fused[1]["loss"], rel=1e-6)
  assert a["loss"] == pytest.approx(b["loss"], rel=5e-3)
  for x, y in zip(a["norm"], b["norm"]):
    assert x == pytest.approx(y, rel=1e-2, abs=1e-3)
  for x, y in zip(a["first"], b["first"]):
    assert x == pytest.approx(y, rel=2e-2, abs=2e-3)


def test_tensor_parallel_graph_decoder_matches_one_gpu(tmp_path):
  """The captured decode step with sharded weights, all-reduce sites over peer memory and
  gathered logits gives the beams of the single-GPU decoder; both model ranks agree exactly."""
  _need_two()
  two = _run_ranks("tp_decode", tmp_path / "tp", n=2)
  one = _run_ranks("tp_decode", tmp_path / "one", n=1)
  assert two[0]["tp"] == 2 and one[0]["tp"] == 1
  assert two[0]["seqs"] == two[1]["seqs"] and two[0]["scores"] == two[1]["scores"]
  assert two[0]["kernels_per_step"] > one[0]["kernels_per_step"]
  same = sum(a == b for a, b in zip(two[0]["seqs"], one[0]["seqs"]))
  assert same >= 6, (two[0]["seqs"], one[0]["seqs"])  # near-ties may reorder under bf16
  for a, b in zip(two[0]["scores"], one[0]["scores"]):
    assert a == pytest.approx(b, rel=2e-2, abs=0.15)
