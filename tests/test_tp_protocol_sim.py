"""The ordering protocol of the fused tensor-parallel kernels under randomised interleavings,
simulated on the CPU.

What runs for real is the host side: `SymmetricArena` (first-fit allocation, quarantine of
released blocks, epoch counter, alternating inboxes, step-end reset), driven by the same call
sequences the autograd functions of `parallel/tp_fused.py` make. What is simulated is the
device: every rank has a stream of kernels, each kernel is a little state machine that follows
the rules of the CUDA kernels (csrc/gemm_pair_sm100.cu, csrc/elementwise.cu):

  all-gather GEMM, epoch e   raises its rank's "rows ready" word to e, then for every peer waits
                             until that peer's word is >= e and copies the peer's rows;
  reduce-scatter GEMM, e     stores its partial rows into slot `rank` of every rank's inbox,
                             then raises its "scattered" word to e;
  slot sum, e                waits until every peer's "scattered" word is >= e, reads all slots;
  barrier                    leaves when every rank has arrived.

A scheduler picks, at random, which rank's stream makes the next micro-step, so ranks run
arbitrarily far apart, as far as the waits allow. Memory cells carry tags; a kernel that reads
a cell checks that it holds the value the program order promises (not a stale one, not one a
peer has already overwritten for a later call). The two host rules under test are the inbox
double-buffering and the quarantine of released arena blocks; breaking either on purpose makes
the same simulator report a violation, which shows that it would notice.
"""
import random

import pytest
import torch

from t5x_b200.ops import comm
from t5x_b200.parallel import tp_fused


class Violation(AssertionError):
  pass


class _World:
  """Device memory, signal words and barrier counters shared by the simulated ranks."""

  def __init__(self, n):
    self.n = n
    self.arena = [dict() for _ in range(n)]       # offset -> tag of the rows stored there
    self.inbox = [dict() for _ in range(n)]       # (turn, slot) -> tag
    self.rows_ready = [0] * n
    self.scattered = [0] * n
    self.arrived = [0] * n


class _FakeSymmetricBuffer:
  """Stands in for `comm.SymmetricBuffer`: host-visible fields only, barriers become stream ops."""

  def __init__(self, numel, dtype, group, device=None):
    self.group, self.rank, self.world = group, group.rank, group.world.n
    self.tensor = torch.zeros(min(int(numel), 1 << 12), dtype=dtype)
    self.peer_ptrs = list(range(self.world))
    self.pad_ptrs = list(range(self.world))

  def barrier(self, channel=0, spin_limit=0):
    self.group.stream.append(("barrier",))


class _Rank:
  def __init__(self, world, rank):
    self.world, self.rank, self.stream = world, rank, []


def _kernel(world: _World, rank: int, op):
  """Generator for one kernel: yields None after a micro-step, or a predicate to wait on."""
  kind = op[0]
  peers = [p for p in range(world.n) if p != rank]
  if kind == "write_own":
    _, offset, tag = op
    world.arena[rank][offset] = tag
    yield None
  elif kind == "allgather":
    _, offset, epoch, call = op
    world.rows_ready[rank] = epoch
    yield None
    random.shuffle(peers)
    for p in peers:
      yield lambda p=p: world.rows_ready[p] >= epoch
      got = world.arena[p].get(offset)
      if got != ("rows", call, p):
        raise Violation(f"rank {rank}, all-gather call {call}: peer {p}'s rows at offset "
                        f"{offset} hold {got}")
      yield None
  elif kind == "reducescatter":
    _, turn, epoch, call = op
    for p in random.sample(range(world.n), world.n):
      world.inbox[p][(turn, rank)] = ("partial", call, rank)
      yield None
    world.scattered[rank] = epoch
    yield None
  elif kind == "slot_sum":
    _, turn, epoch, call = op
    for p in peers:
      yield lambda p=p: world.scattered[p] >= epoch
    for slot in range(world.n):
      got = world.inbox[rank].get((turn, slot))
      if got != ("partial", call, slot):
        raise Violation(f"rank {rank}, slot sum of call {call}: slot {slot} holds {got}")
      yield None
  elif kind == "barrier":
    world.arrived[rank] += 1
    mine = world.arrived[rank]
    yield lambda: min(world.arrived) >= mine
  else:
    raise ValueError(kind)


def _host_program(ar, stream, program, steps):
  """Enqueues, for one rank, the kernels of `steps` training steps of `program` (a list of
  'ag', 'ag_nograd', 'rs'), calling the arena exactly as the autograd functions do."""
  call = 0
  for _ in range(steps):
    kept = []
    for what in program:
      call += 1
      if what in ("ag", "ag_nograd"):
        blk = ar.alloc(4096)
        stream.append(("write_own", blk.offset, ("rows", call, ar.rank)))
        stream.append(("allgather", blk.offset, ar.next_epoch(), call))
        if what == "ag_nograd":
          blk.release()
        else:
          kept.append(blk)
      else:
        ar.next_inbox(1024)
        turn = ar._inbox_turn
        epoch = ar.next_epoch()
        stream.append(("reducescatter", turn, epoch, call))
        stream.append(("slot_sum", turn, epoch, call))
        ar.peers_are_past()
    for blk in reversed(kept):  # the backward pass gives the gathered activations back
      blk.release()
    ar.end_step()


def _simulate(n, program, steps, seed, monkeypatch, arena_bytes=16 * 4096):
  random.seed(seed)
  world = _World(n)
  ranks = [_Rank(world, r) for r in range(n)]
  monkeypatch.setattr(comm, "SymmetricBuffer", _FakeSymmetricBuffer)
  monkeypatch.setattr(torch.cuda, "synchronize", lambda *a, **k: None)
  monkeypatch.setattr(tp_fused.dist, "barrier", lambda *a, **k: None)
  for rk in ranks:
    ar = tp_fused.SymmetricArena(arena_bytes, rk)
    rk.stream.clear()  # set-up barriers are not part of the steps
    _host_program(ar, rk.stream, program, steps)
  position = [0] * n
  running = [None] * n
  waiting = [None] * n
  while True:
    runnable = []
    for r in range(n):
      if running[r] is None and position[r] < len(ranks[r].stream):
        running[r] = _kernel(world, r, ranks[r].stream[position[r]])
        position[r] += 1
      if running[r] is not None and (waiting[r] is None or waiting[r]()):
        runnable.append(r)
    if not runnable:
      if all(g is None for g in running):
        return
      raise Violation(f"deadlock: ranks wait at stream positions {position}")
    r = random.choice(runnable)
    waiting[r] = None
    try:
      waiting[r] = next(running[r])
    except StopIteration:
      running[r] = None


PROGRAMS = [
    ["ag", "rs", "ag", "rs"],                          # one layer, forward
    ["ag_nograd", "ag_nograd", "rs", "ag_nograd", "rs"],  # evaluation: blocks released at once
    ["ag", "ag", "rs", "rs", "ag_nograd", "ag", "rs"],
]


@pytest.mark.parametrize("program", PROGRAMS)
@pytest.mark.parametrize("n", [2, 4])
def test_no_stale_or_overwritten_reads_under_random_interleavings(program, n, monkeypatch):
  for seed in range(40):
    _simulate(n, program, steps=3, seed=seed, monkeypatch=monkeypatch)


def test_arena_pressure_falls_back_to_a_barrier(monkeypatch):
  # room for two blocks only: the third allocation has to wait for proof behind a barrier
  for seed in range(20):
    _simulate(3, ["ag_nograd", "ag_nograd", "ag_nograd", "rs"], steps=2, seed=seed,
              monkeypatch=monkeypatch, arena_bytes=2 * 4096)


def _finds_violation(n, program, monkeypatch, seeds=200):
  for seed in range(seeds):
    try:
      _simulate(n, program, steps=2, seed=seed, monkeypatch=monkeypatch)
    except Violation:
      return True
  return False


def test_simulator_notices_a_single_buffered_inbox(monkeypatch):
  original = tp_fused.SymmetricArena.next_inbox

  def one_buffer(self, nbytes):
    box = original(self, nbytes)
    self._inbox_turn = 0
    return box

  monkeypatch.setattr(tp_fused.SymmetricArena, "next_inbox", one_buffer)
  assert _finds_violation(3, ["rs", "rs", "rs"], monkeypatch)


def test_simulator_notices_blocks_freed_without_quarantine(monkeypatch):
  def free_at_once(self):
    ar, self.arena = self.arena, None
    if ar is not None and self.generation == ar.generation:
      ar._free(self.offset, self.size)

  monkeypatch.setattr(tp_fused._Block, "release", free_at_once)
  assert _finds_violation(3, ["ag_nograd", "ag_nograd", "ag_nograd"], monkeypatch)
