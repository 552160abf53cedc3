"""The Luporax design in the engine against its plain implementation (tests/plain_luporax.py): every way of cutting
requests into steps, in float32 and bfloat16, on configurations that differ in every size, in the order of their layers
and in what is there at all; long decoding over page borders with the recurrent states and the shifts running for
hundreds of steps; pages and state slots used again; greedy generation through the entry point and its scheduler."""
import copy

import numpy as np
import pytest
import torch

import plain_luporax as plain
import replay_cases as rc
from gpu_helpers import DEV

pytestmark = pytest.mark.gpu

LENGTHS = {"A": (5, 17, 33, 100, 64, 128, 41, 65, 1, 2), "B": (1, 9, 40, 71, 130, 65, 200, 2), "C": (130, 70, 300, 64, 200, 65, 257),
           "D": (3, 50, 129, 70, 1, 16)}
PAGES = {"A": 16, "B": 16, "C": 64, "D": 16}
# bfloat16, as fractions of the root mean square of the plain logits: rounding every product to bfloat16 moves a row by a
# few hundredths of that.  A router's close call, decided the other way after rounding, moves single rows by more (an
# expert is exchanged for its neighbour), which is why one row in twenty may pass the bound; a lost state, a shift from a
# wrong row or a key read from a wrong page moves most rows by tenths, and shows in the float32 runs, which take the same
# path through the engine and allow nothing.
BF16_MEAN, BF16_BOUND, BF16_CAP = 0.04, 0.12, 0.6


@pytest.fixture(scope="module")
def luporax_dirs(tmp_path_factory):
  made = {}

  def get(tag):
    if tag not in made:
      made[tag] = plain.make_model_dir(plain.CONFIGS[tag], str(tmp_path_factory.mktemp(f"luporax_{tag}")), seed=61 + len(made))
    return made[tag]

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
  size = float(np.sqrt(np.mean([float(r.pow(2).mean()) for r in ref.values()])))
  if dtype == "float32":
    rc.compare(got, ref, 3e-4 * max(1.0, size), what, check_argmax_margin=2e-3 * max(1.0, size))
    return
  assert got, "nothing was compared"
  errs = []
  for key, row in sorted(got.items()):
    assert np.isfinite(row).all(), f"{what}: request {key[0]} position {key[1]}: logits are not finite"
    d = row - ref[key[0]][key[1]].numpy()
    errs.append(float(np.sqrt(((d - d.mean()) ** 2).mean())) / size)       # root mean square of the centred difference
    assert errs[-1] <= BF16_CAP, f"{what}: request {key[0]} position {key[1]}: the row differs by {errs[-1]:.3f}"
  errs = np.array(errs)
  assert errs.mean() <= BF16_MEAN, f"{what}: rows differ by {errs.mean():.4f} on average"
  assert (errs > BF16_BOUND).sum() <= max(1, 0.05 * len(errs)), f"{what}: {(errs > BF16_BOUND).sum()} of {len(errs)} rows differ by more than {BF16_BOUND}"
  rc.log_worst(what, float(errs.max()), ref)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["A", "B", "C", "D"])
@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed", "preempted"])
def test_every_cut_gives_the_plain_logits(luporax_dirs, dtype, tag, cut):
  d = luporax_dirs(tag)
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
  compare(got, ref, dtype, f"luporax {tag}/{dtype}/{cut}")
  runner.cache.check_invariants()
  assert runner.cache.free_pages() == [g.num_pages for g in runner.cache.paged_groups]
  runner.runner.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["A", "B"])
def test_long_decoding_over_page_borders(luporax_dirs, dtype, tag):
  """Twelve tokens as a prompt, then 250 tokens one by one: the recurrent states and the shifts' rows run over 260 steps,
  the attention reads every earlier key over dozens of page borders (pages of 8), and a second request - portions of three
  tokens, then single ones - runs beside the first from step 100 on."""
  d = luporax_dirs(tag)
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
  compare(got, ref, dtype, f"luporax long decode {tag}/{dtype}")
  runner.cache.check_invariants()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_prompts_whole_and_in_large_portions(luporax_dirs, dtype):
  """Prompts of 1300 and 700 tokens in one step each, then the first in portions of 600: in bfloat16 such steps take the
  recurrences' form for long portions (prepared, then walked in stretches side by side), the library products of the
  gates' parts and the tensor-core attention over dozens of key tiles; the states they leave carry on into single tokens."""
  d = luporax_dirs("C")
  reqs = rc.make_requests(plain.CONFIGS["C"]["vocab"], (1300, 700), seed=17)
  ref = reference(d, reqs)
  a, b = reqs["r0"], reqs["r1"]
  want = lambda lo, hi: list(range(0, hi - lo, 37)) + [hi - lo - 1]
  trace = [{"step": 0, "entries": [{"id": "r0", "tokens": a[:1290], "want": want(0, 1290)}], "end": []}]
  trace += [{"step": 1 + j, "entries": [{"id": "r0", "tokens": [a[1290 + j]], "want": [0]}], "end": ["r0"] if j == 9 else []} for j in range(10)]
  trace.append({"step": 11, "entries": [{"id": "r1", "tokens": b[:600], "want": want(0, 600)}], "end": []})
  trace.append({"step": 12, "entries": [{"id": "r1", "tokens": b[600:], "want": want(600, 700)}], "end": ["r1"]})
  runner = runner_for(d, dtype, 1344, 64)
  got = rc.run_in_process(runner, trace)
  compare(got, ref, dtype, f"luporax long prompts/{dtype}")
  runner.cache.check_invariants()
  runner.runner.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_state_slot_that_is_used_again_starts_from_zero(luporax_dirs, dtype):
  """One state slot and pages for one request: six requests one after the other, each ended before the next comes, the
  third of them cut off in the middle of its prompt.  Every one finds the recurrent states and the shifts' rows at zero
  and its own keys only."""
  d = luporax_dirs("A")
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
  compare(got, ref, dtype, f"luporax slots used again/{dtype}")
  runner.cache.check_invariants()
  assert runner.cache.free_pages() == [g.num_pages for g in runner.cache.paged_groups]


# Weights that single out one key: with a bias of about -9 on every head a key counts only if its score is large, and a
# scale of 1.2 on normed queries and keys spreads the scores of 600 keys over tens of units, so that a position's output is
# the values of a handful of keys, as often hundreds of tokens back as near.  A key read from a wrong page or a wrong
# position, or a cap left out, moves the row as a whole.  The recurrent layer beside it forgets next to nothing.
def peaky_model(folder):
  cfg = {"architecture": "Luporax", "vocab": 200, "width": 64, "norm": {"eps": 1e-5}, "residual_mult": 0.9, "logit_scale": 0.2, "layers": [
    plain.attention(2, 1, 32, 48, 16, 10000.0, 1.2, 25.0, plain.moe(32, 1.0, 4, 2, (16, 1.0))),
    plain.mingru_layer(24, None)]}
  W = plain.make_model(cfg, 77)
  W["l0.mix.pb"] = torch.full_like(W["l0.mix.pb"], -9.0)
  W["l1.mix.z.b"] = torch.full_like(W["l1.mix.z.b"], -7.0)
  return plain.write_model(cfg, W, folder), cfg


@pytest.mark.parametrize("cut", ["whole", "tail", "portions"])
def test_far_keys_stand_out_in_prompts_and_in_decoding(tmp_path, cut):
  d, cfg = peaky_model(str(tmp_path / "peaky"))
  reqs = rc.make_requests(cfg["vocab"], (600, 333), seed=6)
  ref = reference(d, reqs)
  trace = {"whole": rc.whole, "tail": lambda r: rc.tail_one_by_one(r, 70), "portions": rc.portions}[cut](reqs)
  runner = runner_for(d, "float32", 640, 16)
  got = rc.run_in_process(runner, trace)
  compare(got, ref, "float32", f"luporax peaky/{cut}")
  runner.cache.check_invariants()


@pytest.mark.skipif(DEV == "cpu", reason="a property of the CUDA kernels' order of sums, not of the CPU statements")
@pytest.mark.parametrize("tag", ["A", "B"])
def test_float32_logits_do_not_depend_on_the_cut(luporax_dirs, tag):
  """In float32 a position's logits come out the same to the last bit however the request was cut and whatever else was
  in the batch: every sum of the 32-bit path runs in an order that depends on the position alone."""
  d = luporax_dirs(tag)
  reqs = rc.make_requests(plain.CONFIGS[tag]["vocab"], (70, 33, 90, 41), seed=3)
  whole = rc.run_in_process(runner_for(d, "float32", 128, 16), rc.whole(reqs))
  for name, trace in (("portions", rc.portions(reqs)), ("mixed", rc.mixed(reqs, 224, seed=4, granule=16))):
    got = rc.run_in_process(runner_for(d, "float32", 224, 16), trace)
    for key, row in got.items():
      assert np.array_equal(row, whole[key[:2]]), f"{name}: request {key[0]} position {key[1]} differs in its bits"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["A", "C"])
def test_greedy_generation_through_the_engine(luporax_dirs, dtype, tag):
  """``LLMEngine.generate``: the scheduler admits, cuts the prompts into portions under a small token budget, decodes from
  CUDA graphs; more requests than slots, so state slots and pages are used again."""
  from miniinfer_b200 import LLMEngine, SamplingParams
  d = luporax_dirs(tag)
  W, cfg = plain.read_weights(d), plain.read_config(d)
  g = torch.Generator().manual_seed(21)
  prompts = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (3, 45, 18, 70, 9, 31)]
  n_new = 40
  page = PAGES[tag]
  eng = LLMEngine(d, dtype=dtype, device=DEV, page_size=page, num_pages=3 * (128 // page), max_num_seqs=3, max_model_len=128,
                  max_num_batched_tokens=32)
  outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=n_new, ignore_eos=True))
  size = float(plain.forward(cfg, W, prompts[1]).pow(2).mean().sqrt())
  for prompt, out in zip(prompts, outs):
    ids = out["token_ids"]
    assert len(ids) == n_new
    # every token is the plain implementation's choice for the text so far, or within rounding of it
    seq, odd = list(prompt), 0
    for t in ids:
      row = plain.forward(cfg, W, seq)[-1]
      odd += float(row.max() - row[t]) > (1e-3 if dtype == "float32" else 2 * BF16_BOUND) * size
      seq.append(t)
    assert odd <= (0 if dtype == "float32" else 0.05 * n_new), f"{odd} of {n_new} tokens are not what the plain logits allow"
  if DEV != "cpu":
    eng.runner.check_status()
    assert eng.runner.num_graphs() > 0


@pytest.mark.skipif(DEV == "cpu", reason="the command line runs on a CUDA device")
def test_command_line_and_trace_program(luporax_dirs, tmp_path):
  """`main.py` generates from a Luporax folder, and `bin/trace_run` - a process of its own that picks the model by its
  configuration - replays a mixed trace in both dtypes."""
  import json
  import os
  import subprocess
  import sys
  root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
  d = luporax_dirs("B")
  W, cfg = plain.read_weights(d), plain.read_config(d)
  proc = subprocess.run([sys.executable, os.path.join(root, "main.py"), "--model", d, "--prompt-ids", "5,17,3,199", "--max-tokens", "6",
                         "--temperature", "0", "--dtype", "float32", "--max-model-len", "64", "--page-size", "16"],
                        capture_output=True, text=True, timeout=900)
  assert proc.returncode == 0, proc.stderr[-3000:]
  assert str(plain.generate(cfg, W, [5, 17, 3, 199], 6)) in proc.stdout
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
