"""The Famupel design in the engine against its plain implementation (tests/plain_famupel.py): every way of cutting
requests into steps, in float32 and bfloat16, on configurations that differ in every size, in the order of their layers
and in whether there are residual streams at all; long decoding over page borders with the recurrent states running for
hundreds of steps; pages and state slots used again; greedy generation through the entry point and its scheduler."""
import copy

import numpy as np
import pytest
import torch

import plain_famupel as plain
import replay_cases as rc
from gpu_helpers import DEV

pytestmark = pytest.mark.gpu

LENGTHS = {"A": (5, 17, 33, 100, 64, 128, 41, 65, 1, 2), "B": (1, 9, 40, 71, 130, 65, 200, 2), "C": (130, 70, 300, 64, 200, 65, 257)}
PAGES = {"A": 16, "B": 16, "C": 64}
# bfloat16: logits of these models have a root mean square near 1; rounding every product to bfloat16 moves a row by a few
# hundredths on average, and the matrix states carry the rounding of every earlier token.  A lost state, a decay applied
# to the wrong rows or a stream mixed the wrong way round moves most rows by tenths, and shows in the float32 runs, which
# take the same path through the engine and allow nothing.
BF16_MEAN, BF16_BOUND, BF16_CAP = 0.05, 0.15, 0.45      # the mean over all rows; what one row in twenty may pass; what none may


def config_for(tag, dtype="float32"):
  """C has a head whose decay is 0: its read-out is (q_t . k_t) v_t, and the norm behind it leaves the sign of q_t . k_t
  times the direction of v_t - a coin toss wherever the product is near zero, so rounding to bfloat16 turns single rows
  over.  The float32 runs keep that head; the bfloat16 runs forget a little less fast.  (The kernel alone is held to a
  decay of 0 in both dtypes, from the same rounded inputs.)"""
  cfg = plain.CONFIGS[tag]
  if tag == "C" and dtype == "bfloat16":
    cfg = copy.deepcopy(cfg)
    cfg["layers"][1]["mixer"]["right"]["decay"] = [1.0, 0.25]
  return cfg


@pytest.fixture(scope="module")
def famupel_dirs(tmp_path_factory):
  made = {}

  def get(tag, dtype="float32"):
    cfg = config_for(tag, dtype)
    key = (tag, cfg is plain.CONFIGS[tag])
    if key not in made:
      made[key] = plain.make_model_dir(cfg, str(tmp_path_factory.mktemp(f"famupel_{tag}")), seed=41 + len(made), ranks=plain.RANKS[tag])
    return made[key]

  return get


_refs = {}


def reference(model_dir, reqs):
  key = (model_dir, tuple(sorted(reqs)), tuple(len(v) for v in reqs.values()))
  if key not in _refs:
    W, cfg = plain.read_weights(model_dir), plain.read_config(model_dir)
    with torch.no_grad():
      _refs[key] = {rid: plain.forward(cfg, W, ids) for rid, ids in reqs.items()}
  return _refs[key]


def runner_for(model_dir, dtype, max_tokens, page, max_requests=4):
  from miniinfer_b200.engine.replay import TraceRunner
  return TraceRunner(model_dir, dtype, max_tokens, device=DEV, page_size=page, max_requests=max_requests)


def compare(got, ref, dtype, what):
  if dtype == "float32":
    rc.compare(got, ref, 3e-4, what, check_argmax_margin=2e-3)
    return
  assert got, "nothing was compared"
  errs = []
  for key, row in sorted(got.items()):
    assert np.isfinite(row).all(), f"{what}: request {key[0]} position {key[1]}: logits are not finite"
    d = row - ref[key[0]][key[1]].numpy()
    errs.append(float(np.sqrt(((d - d.mean()) ** 2).mean())))       # root mean square of the centred difference
    assert errs[-1] <= BF16_CAP, f"{what}: request {key[0]} position {key[1]}: the row differs by {errs[-1]:.3f}"
  errs = np.array(errs)
  assert errs.mean() <= BF16_MEAN, f"{what}: rows differ by {errs.mean():.4f} on average"
  assert (errs > BF16_BOUND).sum() <= max(1, 0.05 * len(errs)), f"{what}: {(errs > BF16_BOUND).sum()} of {len(errs)} rows differ by more than {BF16_BOUND}"
  rc.log_worst(what, float(errs.max()), ref)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["A", "B", "C"])
@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed", "preempted"])
def test_every_cut_gives_the_plain_logits(famupel_dirs, dtype, tag, cut):
  d = famupel_dirs(tag, dtype)
  page = PAGES[tag]
  reqs = rc.make_requests(plain.CONFIGS[tag]["vocab"], LENGTHS[tag], seed=5)
  ref = reference(d, reqs)
  longest = rc.round_up(max(LENGTHS[tag]), page)
  if cut in ("mixed", "preempted"):
    budget = longest + 2 * rc.round_up(70, page)      # requests wait for pages that others give back
    trace = rc.mixed(reqs, budget, seed=1, granule=page, preempt=cut == "preempted")
    assert max(len(r["entries"]) for r in trace) >= 2
  else:
    budget = longest
    trace = {"whole": rc.whole, "tail": rc.tail_one_by_one, "portions": rc.portions}[cut](reqs)
  runner = runner_for(d, dtype, budget, page)
  got = rc.run_in_process(runner, trace)
  compare(got, ref, dtype, f"famupel {tag}/{dtype}/{cut}")
  runner.cache.check_invariants()
  assert runner.cache.free_pages() == [g.num_pages for g in runner.cache.paged_groups]
  runner.runner.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["A", "B"])
def test_long_decoding_over_page_borders(famupel_dirs, dtype, tag):
  """Twelve tokens as a prompt, then 250 tokens one by one: the matrix states run over 260 steps, the attention of the
  pairs reads every earlier key over dozens of page borders (pages of 8), and a second request - portions of three
  tokens, then single ones - runs beside the first from step 100 on."""
  d = famupel_dirs(tag)
  reqs = rc.make_requests(plain.CONFIGS[tag]["vocab"], (262, 150), seed=9)
  ref = reference(d, reqs)
  a, b = reqs["r0"], reqs["r1"]
  trace = [{"step": 0, "entries": [{"id": "r0", "tokens": a[:12], "want": list(range(12))}], "end": []}]
  pos_b = 0
  for j in range(12, len(a)):
    entries = [{"id": "r0", "tokens": [a[j]], "want": [0]}]
    if j >= 100 and pos_b < len(b):
      n = 3 if pos_b < 30 else 1
      entries.append({"id": "r1", "tokens": b[pos_b:pos_b + n], "want": list(range(len(b[pos_b:pos_b + n])))})
      pos_b += n
    trace.append({"step": len(trace), "entries": entries, "end": []})
  trace[-1]["end"] = ["r0", "r1"]
  runner = runner_for(d, dtype, 512, 8)
  got = rc.run_in_process(runner, trace)
  got = {k: v for k, v in got.items() if k[0] == "r0" or k[1] < pos_b}
  compare(got, ref, dtype, f"famupel long decode {tag}/{dtype}")
  runner.cache.check_invariants()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_state_slot_that_is_used_again_starts_from_zero(famupel_dirs, dtype):
  """One state slot and pages for one request: six requests one after the other, each ended before the next comes, the
  third of them cut off in the middle of its prompt.  Every one finds the matrix states at zero and its own keys only."""
  d = famupel_dirs("A")
  reqs = rc.make_requests(plain.CONFIGS["A"]["vocab"], (40, 64, 50, 7, 33, 2), seed=12)
  ref = reference(d, reqs)
  runner = runner_for(d, dtype, 64, 16, max_requests=1)
  trace = []
  for rid, ids in reqs.items():
    if rid == "r2":                            # given up half way: what it wrote stays behind in slot and pages
      trace.append({"step": len(trace), "entries": [{"id": "x", "tokens": ids[:25], "want": []}], "end": ["x"]})
    cut = max(1, len(ids) // 3)
    trace.append({"step": len(trace), "entries": [{"id": rid, "tokens": ids[:cut], "want": list(range(cut))}], "end": []})
    if cut < len(ids):
      trace.append({"step": len(trace), "entries": [{"id": rid, "tokens": ids[cut:], "want": list(range(len(ids) - cut))}], "end": [rid]})
    else:
      trace[-1]["end"] = [rid]
  got = rc.run_in_process(runner, trace)
  got = {k: v for k, v in got.items() if k[0] != "x"}
  assert len(got) == sum(len(v) for v in reqs.values())
  compare(got, ref, dtype, f"famupel slots used again/{dtype}")
  runner.cache.check_invariants()
  assert runner.cache.free_pages() == [g.num_pages for g in runner.cache.paged_groups]


# Scores that single out one key: after the norm over the whole projection a query and a key head have a length near
# sqrt(dim), so a scale of 1.5 spreads the scores of 600 keys over tens of units and nearly all of a position's weight
# falls on one key, as often hundreds of tokens back as near.  The retention beside it forgets nothing (decay 1) or
# next to nothing.  A key read from a wrong page or a wrong position moves the row as a whole.
PEAKY = {"architecture": "Famupel", "vocab": 200, "width": 64, "norm": {"eps": 1e-5}, "streams": 2, "layers": [
  plain.pair(plain.left_of(2, 1, 32, 48, plain.rot_of(16, 10000.0), 1.5), plain.right_of(2, 16, 16, plain.rot_of(8, 100.0), [1.0, 0.9995]),
             1.0, 0.5, plain.dense(64)),
  plain.gla(2, 16, 16, 64.0, None)]}


@pytest.mark.parametrize("cut", ["whole", "tail", "portions"])
def test_far_keys_stand_out_in_prompts_and_in_decoding(tmp_path, cut):
  d = plain.make_model_dir(PEAKY, str(tmp_path / "peaky"), seed=77, ranks={1: 4})
  reqs = rc.make_requests(PEAKY["vocab"], (600, 333), seed=6)
  ref = reference(d, reqs)
  trace = {"whole": rc.whole, "tail": lambda r: rc.tail_one_by_one(r, 70), "portions": rc.portions}[cut](reqs)
  runner = runner_for(d, "float32", 640, 16)
  got = rc.run_in_process(runner, trace)
  rc.compare(got, ref, 3e-4, f"famupel peaky/{cut}")
  runner.cache.check_invariants()


@pytest.mark.skipif(DEV == "cpu", reason="a property of the CUDA kernels' order of sums, not of the CPU statements")
@pytest.mark.parametrize("tag", ["A", "B"])
def test_float32_logits_do_not_depend_on_the_cut(famupel_dirs, tag):
  """In float32 a position's logits come out the same to the last bit however the request was cut and whatever else was
  in the batch: every sum of the 32-bit path runs in an order that depends on the position alone."""
  d = famupel_dirs(tag)
  reqs = rc.make_requests(plain.CONFIGS[tag]["vocab"], (70, 33, 90, 41), seed=3)
  whole = rc.run_in_process(runner_for(d, "float32", 128, 16), rc.whole(reqs))
  for name, trace in (("portions", rc.portions(reqs)), ("mixed", rc.mixed(reqs, 224, seed=4, granule=16))):
    got = rc.run_in_process(runner_for(d, "float32", 224, 16), trace)
    for key, row in got.items():
      assert np.array_equal(row, whole[key[:2]]), f"{name}: request {key[0]} position {key[1]} differs in its bits"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["A", "B"])
def test_greedy_generation_through_the_engine(famupel_dirs, dtype, tag):
  """``LLMEngine.generate``: the scheduler admits, cuts the prompts into portions under a small token budget, decodes from
  CUDA graphs; more requests than slots, so state slots and pages are used again."""
  from miniinfer_b200 import LLMEngine, SamplingParams
  d = famupel_dirs(tag)
  W, cfg = plain.read_weights(d), plain.read_config(d)
  g = torch.Generator().manual_seed(21)
  prompts = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (3, 45, 18, 70, 9, 31)]
  n_new = 40
  eng = LLMEngine(d, dtype=dtype, device=DEV, page_size=16, num_pages=24, max_num_seqs=3, max_model_len=128,
                  max_num_batched_tokens=32)
  outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=n_new, ignore_eos=True))
  for prompt, out in zip(prompts, outs):
    ids = out["token_ids"]
    assert len(ids) == n_new
    if dtype == "float32":
      assert ids == plain.generate(cfg, W, prompt, n_new)
    else:
      # every token is the plain implementation's choice for the text so far, or within the bound of it
      seq, odd = list(prompt), 0
      for t in ids:
        row = plain.forward(cfg, W, seq)[-1]
        odd += float(row.max() - row[t]) > 2 * BF16_BOUND
        seq.append(t)
      assert odd <= 0.05 * n_new, f"{odd} of {n_new} bfloat16 tokens are not what the plain logits allow"
  if DEV != "cpu":
    eng.runner.check_status()
    assert eng.runner.num_graphs() > 0


@pytest.mark.skipif(DEV == "cpu", reason="the command line runs on a CUDA device")
def test_command_line_and_trace_program(famupel_dirs, tmp_path):
  """`main.py` generates from a Famupel folder, and `bin/trace_run` - a process of its own that picks the model by its
  configuration - replays a mixed trace in both dtypes."""
  import json
  import os
  import subprocess
  import sys
  root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
  d = famupel_dirs("B")
  W, cfg = plain.read_weights(d), plain.read_config(d)
  proc = subprocess.run([sys.executable, os.path.join(root, "main.py"), "--model", d, "--prompt-ids", "5,17,3,200", "--max-tokens", "6",
                         "--temperature", "0", "--dtype", "float32", "--max-model-len", "64", "--page-size", "16"],
                        capture_output=True, text=True, timeout=900)
  assert proc.returncode == 0, proc.stderr[-3000:]
  assert str(plain.generate(cfg, W, [5, 17, 3, 200], 6)) in proc.stdout
  reqs = rc.make_requests(cfg["vocab"], (70, 9, 130), seed=2)
  ref = reference(d, reqs)
  trace = rc.mixed(reqs, 256, seed=3)
  for dtype in ("float32", "bfloat16"):
    out = tmp_path / dtype
    proc = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", d, "--dtype", dtype, "--out", str(out), "--max-tokens", "256"],
                          input="\n".join(json.dumps(r) for r in trace) + "\n", capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    assert [l for l in proc.stdout.split("\n") if l.startswith("done")] == [f"done {r['step']}" for r in trace]
    outputs = {r["step"]: np.fromfile(out / f"{r['step']}.f32", dtype="<f4").reshape(-1, cfg["vocab"])
               for r in trace if sum(len(e["want"]) for e in r["entries"])}
    compare(rc.collect(trace, outputs), ref, dtype, f"trace program {dtype}")
