"""Failure detection and recovery, exercised from the host only: ranks are CPU processes over
gloo, failures are exceptions, missing ranks, damaged files and signals. No test here touches a
GPU.

  * a rank that never reaches a host barrier / dies inside a checkpoint save turns into a
    `HostSyncError` on the ranks that wait for it, within the timeout;
  * unfinished `checkpoint_N.tmp-*` directories are invisible to step discovery and removed by
    the next save;
  * a damaged newest checkpoint (index file gone, array chunk truncated) makes a resuming run
    fall back to the checkpoint before it;
  * SIGTERM stops training at a step boundary with an emergency checkpoint, and the resumed run
    continues on the loss curve of an uninterrupted run;
  * the same seed gives the same losses twice.
"""
import glob
import os
import signal
import socket
import sys
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from t5x_b200 import checkpoints
from t5x_b200 import gin
from t5x_b200 import train as train_lib
from t5x_b200 import trainer as trainer_lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TASK = "synthetic_span_corruption"


def _free_port():
  s = socket.socket()
  s.bind(("127.0.0.1", 0))
  p = s.getsockname()[1]
  s.close()
  return p


@pytest.fixture(autouse=True)
def _fresh_gin():
  gin.clear_config(clear_constants=True)
  yield
  gin.clear_config(clear_constants=True)


# ----------------------------------------------------------------------------
# ranks that go missing
# ----------------------------------------------------------------------------
def _init(rank, world, port):
  sys.path.insert(0, ROOT)
  os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                    WORLD_SIZE=str(world))
  dist.init_process_group("gloo", rank=rank, world_size=world)
  from t5x_b200.parallel import state as pstate
  pstate.setup_mesh(model_size=1, device=torch.device("cpu"))
  return pstate


def _barrier_worker(rank, world, port, out_dir):
  pstate = _init(rank, world, port)
  pstate.host_barrier("both ranks are here", timeout_s=30)
  if rank == 1:
    time.sleep(6)  # never joins the second barrier; leaves without an error
    return
  tick = time.time()
  try:
    pstate.host_barrier("rank 1 never comes", timeout_s=2)
    outcome = "returned"
  except pstate.HostSyncError as e:
    outcome = f"error after {time.time() - tick:.1f}s: {e}"
  with open(os.path.join(out_dir, "rank0.txt"), "w") as f:
    f.write(outcome)


def test_host_barrier_times_out_instead_of_hanging(tmp_path):
  mp.spawn(_barrier_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
  outcome = open(tmp_path / "rank0.txt").read()
  assert outcome.startswith("error after"), outcome
  assert "rank 1 never comes" in outcome
  assert float(outcome.split()[2][:-2]) < 5.5


def _tiny_state():
  from t5x_b200 import adafactor, models, train_state as ts_lib
  from t5x_b200.data import vocabularies
  from t5x_b200.models import base
  from t5x_b200.models.t5 import network
  cfg = network.T5Config(vocab_size=64, dtype="float32", emb_dim=32, num_heads=2,
                         num_encoder_layers=1, num_decoder_layers=1, head_dim=16, mlp_dim=64,
                         mlp_activations=("gelu", "linear"), dropout_rate=0.0)
  torch.manual_seed(0)
  module = network.Transformer(cfg)
  vocab = vocabularies.PassThroughVocabulary(64)
  model = models.EncoderDecoderModel(module, vocab, vocab, adafactor.Adafactor())
  return ts_lib.FlaxOptimTrainState.create(
      model.optimizer_def, {"params": base.module_param_tree(module),
                            "params_axes": base.module_param_axes(module)})


def _save_worker(rank, world, port, ckpt_dir, out_dir):
  pstate = _init(rank, world, port)
  os.environ["T5X_B200_HOST_SYNC_TIMEOUT_S"] = "3"
  from t5x_b200 import partitioning
  state = _tiny_state()
  ck = checkpoints.Checkpointer(state, partitioning.PjitPartitioner(num_partitions=1), ckpt_dir)
  if rank == 1:
    # this rank "crashes" while writing its arrays: it never reaches the barrier after them
    def boom(*a, **k):
      raise OSError("disk went away")
    ck._write_state_to_tensorstore = boom
  try:
    ck.save(state)
    outcome = "saved"
  except pstate.HostSyncError as e:
    outcome = f"sync error: {e}"
  except OSError as e:
    outcome = f"io error: {e}"
  with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
    f.write(outcome)


def test_rank_that_dies_inside_a_save_fails_the_save_on_the_others(tmp_path):
  ckpt_dir, out_dir = str(tmp_path / "ckpt"), str(tmp_path / "out")
  os.makedirs(ckpt_dir)
  os.makedirs(out_dir)
  mp.spawn(_save_worker, args=(2, _free_port(), ckpt_dir, out_dir), nprocs=2, join=True)
  assert open(os.path.join(out_dir, "rank1.txt")).read().startswith("io error")
  r0 = open(os.path.join(out_dir, "rank0.txt")).read()
  assert r0.startswith("sync error") and "tensorstore_write_complete" in r0, r0
  # nothing half-written is visible as a checkpoint; the leftover is a .tmp- directory
  assert checkpoints.all_steps(ckpt_dir) == []
  assert glob.glob(os.path.join(ckpt_dir, "checkpoint_0.tmp-*"))


# ----------------------------------------------------------------------------
# leftovers and damage on disk
# ----------------------------------------------------------------------------
def test_unfinished_tmp_directories_are_ignored_and_cleaned(tmp_path):
  from t5x_b200 import partitioning
  ckpt_dir = str(tmp_path)
  stale = os.path.join(ckpt_dir, "checkpoint_7.tmp-1700000000")
  os.makedirs(stale)
  open(os.path.join(stale, "junk"), "w").write("x")
  assert checkpoints.all_steps(ckpt_dir) == []
  assert checkpoints.latest_step(ckpt_dir) is None
  state = _tiny_state()
  ck = checkpoints.Checkpointer(state, partitioning.PjitPartitioner(num_partitions=1), ckpt_dir)
  ck.save(state)
  assert checkpoints.all_steps(ckpt_dir) == [0]
  assert not os.path.exists(stale)


def _train_args(model_dir, steps, extra=()):
  return (["--gin_file=t5x/examples/t5/t5_1_1/tiny.gin",
           "--gin_file=t5x/configs/runs/pretrain.gin",
           "--gin_file=t5x/examples/t5/local_tiny.gin",
           "--gin.VOCABULARY=@seqio.PassThroughVocabulary()",
           "--gin.seqio.PassThroughVocabulary.size=32128", "--gin.DROPOUT_RATE=0.0",
           f'--gin.MODEL_DIR="{model_dir}"', f'--gin.MIXTURE_OR_TASK_NAME="{TASK}"',
           "--gin.USE_CACHED_TASKS=False", f"--gin.TRAIN_STEPS={steps}",
           "--gin.utils.CheckpointConfig.save=@utils.SaveCheckpointConfig()",
           "--gin.utils.SaveCheckpointConfig.period=2",
           "--gin.utils.SaveCheckpointConfig.save_dataset=True",
           "--gin.train_script.train.eval_period=2",
           "--gin.train_script.train.random_seed=11",
           "--gin.train_script.train.stats_period=1"] + list(extra))


class _Losses(trainer_lib.BaseAction):
  """Records the loss after every stats period."""

  def __init__(self):
    self.values = {}

  def run(self, train_state, metrics_by_task):
    self.values[int(train_state.step)] = float(metrics_by_task["train"]["loss"].value)
    return False


def _run_train(model_dir, steps, **overrides):
  """`train.main` with keyword overrides of `train()` (actions, dataset functions)."""
  from t5x_b200 import gin_utils
  gin.clear_config(clear_constants=True)
  argv = gin_utils.rewrite_gin_args(_train_args(model_dir, steps))
  flags = train_lib.build_flag_parser("").parse_args(argv)
  gin.set_main_module(sys.modules[train_lib.__name__])
  train_lib.parse_gin_from_flags(flags, train_lib._DEFAULT_GIN_SEARCH_PATHS)
  return gin.get_configurable(train_lib.train)(**overrides)


@pytest.mark.parametrize("damage", ["index_missing", "chunk_truncated"])
def test_damaged_newest_checkpoint_falls_back_to_the_previous_one(tmp_path, damage, caplog):
  model_dir = str(tmp_path / "run")
  _run_train(model_dir, 4)
  assert checkpoints.all_steps(model_dir) == [0, 2, 4]
  newest = os.path.join(model_dir, "checkpoint_4")
  if damage == "index_missing":
    os.remove(os.path.join(newest, "checkpoint"))
  else:
    chunks = [p for p in glob.glob(os.path.join(newest, "target.*", "*"))
              if os.path.basename(p) != ".zarray" and os.path.getsize(p) > 64]
    assert chunks
    for p in chunks:
      with open(p, "r+b") as f:
        f.truncate(os.path.getsize(p) // 2)
  losses = _Losses()
  with caplog.at_level("WARNING"):
    last_step, _ = _run_train(model_dir, 6, actions={"TRAIN": [losses]})
  assert last_step == 6
  assert any("trying the previous one" in r.getMessage() for r in caplog.records)
  # the run resumed at step 2 (the newest readable checkpoint), not from scratch
  assert min(losses.values) == 3 and max(losses.values) == 6


# ----------------------------------------------------------------------------
# preemption
# ----------------------------------------------------------------------------
def test_sigterm_writes_an_emergency_checkpoint_and_the_resumed_run_continues_the_curve(tmp_path):
  straight = _Losses()
  _run_train(str(tmp_path / "a"), 6, actions={"TRAIN": [straight]})
  assert sorted(straight.values) == [1, 2, 3, 4, 5, 6]

  class _KillAtStep3(_Losses):
    def run(self, train_state, metrics_by_task):
      super().run(train_state, metrics_by_task)
      if int(train_state.step) == 3:
        os.kill(os.getpid(), signal.SIGTERM)  # handled between steps by the trainer
      return False

  model_dir = str(tmp_path / "b")
  first = _KillAtStep3()
  with pytest.raises(trainer_lib.PreemptionError):
    _run_train(model_dir, 6, actions={"TRAIN": [first]})
  assert 3 in checkpoints.all_steps(model_dir)  # the emergency checkpoint
  second = _Losses()
  last_step, _ = _run_train(model_dir, 6, actions={"TRAIN": [second]})
  assert last_step == 6 and sorted(second.values) == [4, 5, 6]
  resumed = {**first.values, **second.values}
  for step in range(1, 7):
    assert resumed[step] == pytest.approx(straight.values[step], rel=1e-6), step


def test_same_seed_gives_the_same_losses(tmp_path):
  a, b = _Losses(), _Losses()
  _run_train(str(tmp_path / "a"), 3, actions={"TRAIN": [a]})
  _run_train(str(tmp_path / "b"), 3, actions={"TRAIN": [b]})
  assert a.values == b.values and len(a.values) == 3


def test_profile_steps_hook_writes_a_trace_for_the_requested_steps(tmp_path, monkeypatch):
  from t5x_b200.utils import profiling
  assert profiling.parse_step_range("2:4") == (2, 4) and profiling.parse_step_range("3") == (3, 4)
  with pytest.raises(ValueError):
    profiling.parse_step_range("4:2")
  monkeypatch.setenv("T5X_B200_PROFILE_STEPS", "1:3")
  model_dir = str(tmp_path / "run")
  _run_train(model_dir, 4)
  files = sorted(os.path.basename(p) for p in glob.glob(os.path.join(model_dir, "profile", "*")))
  assert files == ["steps_1_3.rank0.kernels.txt", "steps_1_3.rank0.trace.json"]
  assert os.path.getsize(os.path.join(model_dir, "profile", files[1])) > 1000
