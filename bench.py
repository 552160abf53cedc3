#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Default run: the layer sizes of a Qwen3-0.6B-shaped model (28 layers, hidden 1024, 16 query and
8 kv heads of 128, intermediate 3072, vocabulary 151936, tied head) in bfloat16, 8 requests with a
2048-token context each.  A step is one decode step of the whole batch.

One JSON line is printed:
  value      decoded tokens per second of the step function with sampling (CUDA-graph replay, device
             timing with CUDA events around K steps; every step reads weights + cache, far more than L2)
  e2e        the same through ``LLMEngine.step`` - scheduler, pinned-host token/metadata upload, graph
             replay, sampled tokens back to the host - timed around K engine steps
  prefill    one whole 2048-token prompt in one step: tokens/s, ms, fraction of the bf16 tensor peak
  roofline   bytes the decode step must read (every weight once + the cache of the live requests)
             divided by its time, against the measured HBM copy bandwidth
  points     decode tokens/s at batch 1 and 64
  kernels    the dominant kernels of the decode step (the matrix products that stream the weights, the
             attention kernel that streams the cache) and of the prefill step (the matrix products, the
             attention kernel): microseconds per step from CUPTI kernel records of a few further steps,
             the bytes or FLOPs they account for, and the rate that follows against the measured peak

``--shape 8b`` / ``--shape 32b`` run the same measurement at the layer sizes of Qwen3-8B (36 layers) and
Qwen3-32B (64 layers, 4096-token contexts, max_model_len 8192).
"""
import argparse
import gc
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODEL = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=28, hidden_size=1024,
             num_attention_heads=16, num_key_value_heads=8, head_dim=128, intermediate_size=3072, vocab_size=151936,
             rope_theta=1000000.0, rms_norm_eps=1e-6, max_position_embeddings=40960, tie_word_embeddings=True)
# other shapes for --shape: what differs from MODEL
SHAPES = {"0.6b": {},
          "8b": dict(num_hidden_layers=36, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                     intermediate_size=12288, tie_word_embeddings=False),
          "32b": dict(num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, num_key_value_heads=8, head_dim=128,
                      intermediate_size=25600, tie_word_embeddings=False)}
SHAPE_CONTEXT = {"32b": 4096}          # tokens each request holds when decoding starts, where it is not 2048
SHAPE_MAX_MODEL_LEN = {"32b": 8192}
CONTEXT = 2048
GENERATED = 256
MAX_MODEL_LEN = 4096
PREFILL_TOKENS = 2048
PAGE = 64


def peaks():
  path = os.path.join(ROOT, "MEASURED_PEAKS.json")
  if os.path.exists(path):
    with open(path) as f:
      d = json.load(f)
    return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "source": "measured"}
  return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
  """Samples SM clocks and throttle reasons with nvidia-smi while the timed regions run."""

  FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
            "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

  def __init__(self):
    self.samples = []
    self.proc = None
    self.thread = None

  def start(self):
    try:
      self.proc = subprocess.Popen(["nvidia-smi", "--id=0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "25"],
                                   stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
    except OSError:
      return
    self.thread = threading.Thread(target=self._read, daemon=True)
    self.thread.start()

  def _read(self):
    for line in self.proc.stdout:
      parts = [p.strip() for p in line.split(",")]
      if len(parts) == 6:
        self.samples.append(parts)

  def stop(self) -> dict:
    if self.proc is None:
      return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
    self.proc.terminate()
    try:
      self.proc.wait(timeout=5)
    except subprocess.TimeoutExpired:
      self.proc.kill()
    mhz, mx, reasons = [], None, set()
    for s in self.samples:
      try:
        mhz.append(float(s[0]))
        mx = float(s[1])
      except ValueError:
        continue
      for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[2:]):
        if v.lower().startswith("active"):
          reasons.add(name)
    # the median under load: a run that builds models between its timed stretches leaves the GPU idle (at a few hundred
    # MHz) for most of its samples; those that lie below a third of the maximum are idle ones and do not count
    busy = sorted(m for m in mhz if mx and m >= mx / 3.0) or sorted(mhz)
    return {"sm_mhz": busy[len(busy) // 2] if busy else None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(mhz),
            "samples_under_load": len(busy)}


def model_bytes(cfg: dict, layers: int) -> dict:
  H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
  nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
  per_layer = ((nh + 2 * nkv) * hd * H + H * nh * hd + 2 * I * H + H * I) * 2 + (2 * H + 2 * hd) * 4
  head = V * H * 2
  return {"weights": layers * per_layer + head + H * 4, "kv_per_token": layers * 2 * nkv * hd * 2}


def prefill_flops(cfg: dict, layers: int, T: int) -> float:
  H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
  nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
  gemm = 2.0 * T * ((nh + 2 * nkv) * hd * H + H * nh * hd + 2 * I * H + H * I) * layers + 2.0 * V * H
  attn = layers * 2.0 * 2.0 * nh * hd * (T * (T + 1) / 2)
  return gemm + attn


def build_engine(model_dir: str, batch: int):
  from miniinfer_b200 import LLMEngine
  pages = batch * (-(-(CONTEXT + GENERATED + 128) // PAGE)) + 8          # GENERATED covers warm-up + steps (see main)
  pages = max(pages, -(-PREFILL_TOKENS // PAGE) + 8)
  return LLMEngine(model_dir, dtype="bfloat16", device="cuda:0", load_format="random", page_size=PAGE, num_pages=pages,
                   max_num_seqs=max(batch, 1), max_model_len=MAX_MODEL_LEN, max_num_batched_tokens=PREFILL_TOKENS, seed=0)


def fill_context(engine, batch: int, tokens: int, seed: int):
  """Admits `batch` requests and runs their prompts through the step function in portions."""
  import torch
  from miniinfer_b200.engine import StepItem
  g = torch.Generator().manual_seed(seed)
  V = engine.model_config.vocab_size
  ids = []
  for b in range(batch):
    rid = f"bench{b}"
    engine.cache.admit(rid)
    prompt = torch.randint(0, V, (tokens,), generator=g).tolist()
    for s in range(0, tokens, PREFILL_TOKENS):
      engine.runner.step([StepItem(rid, prompt[s:s + PREFILL_TOKENS], ())])
    ids.append(rid)
  torch.cuda.synchronize()
  return ids


def time_decode(engine, batch: int, steps: int, warmup: int) -> dict:
  """K decode steps of the step function with sampling, through the decode CUDA graph."""
  import torch
  from miniinfer_b200.engine import StepItem
  from miniinfer_b200.sampling import Sampler, SamplingParams
  rids = fill_context(engine, batch, CONTEXT, seed=batch)
  params = [SamplingParams(temperature=0.6, max_tokens=GENERATED, ignore_eos=True)] * batch
  tokens_dev = torch.zeros(max(batch, 1), dtype=torch.int32, device="cuda:0")
  last = [1] * batch
  n = [0]

  def one():
    extras = Sampler.pack(params, list(range(batch)), [n[0]] * batch)
    items = [StepItem(r, [t], (0,)) for r, t in zip(rids, last)]
    engine.runner.step_and_sample(items, extras, Sampler.sample, tokens_dev, sampling_pad=Sampler.PAD_ROWS)
    n[0] += 1

  for _ in range(max(warmup, 3)):
    one()
  torch.cuda.synchronize()
  start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  start.record()
  for _ in range(steps):
    one()
  end.record()
  torch.cuda.synchronize()
  ms = start.elapsed_time(end) / steps
  launches = engine.runner.last_launches
  mean_ctx = CONTEXT + max(warmup, 3) + steps / 2.0
  for r in rids:
    engine.cache.release_request(r)
  return {"ms": ms, "tok_s": batch * 1000.0 / ms, "launches_per_step": launches, "mean_ctx": mean_ctx}


def time_e2e(engine, batch: int, steps: int, warmup: int) -> dict:
  """The same decode steps through the Python entry point: host tokens in, host tokens out."""
  import torch
  from miniinfer_b200 import SamplingParams
  g = torch.Generator().manual_seed(100 + batch)
  V = engine.model_config.vocab_size
  # the first requests decode while the later ones' prompts still run, portion by portion
  early = batch * -(-CONTEXT // PREFILL_TOKENS)
  sp = SamplingParams(temperature=0.6, max_tokens=max(warmup, 3) + steps + early + 16, ignore_eos=True)
  for b in range(batch):
    engine.add_request(torch.randint(0, V, (CONTEXT,), generator=g).tolist(), sp)
  while any(r.total_len - r.num_computed != 1 for r in engine.scheduler.running) or engine.scheduler.waiting:
    engine.step()                      # prompts, in portions under the token budget
  for _ in range(max(warmup, 3)):
    engine.step()
  torch.cuda.synchronize()
  s0 = dict(engine.stats)
  t0 = time.perf_counter()
  for _ in range(steps):
    engine.step()
  torch.cuda.synchronize()
  dt = time.perf_counter() - t0
  s1 = dict(engine.stats)
  host = {k[5:-2]: round(1e6 * (s1[k] - s0[k]) / steps, 1) for k in s1 if k.startswith("host_")}
  print(f"e2e host microseconds per step by phase: {host}", file=sys.stderr)
  assert s1["decode_tokens"] - s0["decode_tokens"] == batch * steps, "the timed steps were not pure decode steps"
  while engine.has_unfinished():
    engine.step()
  return {"tok_s": batch * steps / dt, "ms": 1000.0 * dt / steps,
          "h2d": (s1["h2d_bytes"] - s0["h2d_bytes"]) / steps, "d2h": (s1["d2h_bytes"] - s0["d2h_bytes"]) / steps,
          "launches": (s1["launches"] - s0["launches"]) / steps}


def time_prefill(engine, reps: int = 5) -> dict:
  import torch
  from miniinfer_b200.engine import StepItem
  g = torch.Generator().manual_seed(7)
  V = engine.model_config.vocab_size
  times = []
  for i in range(reps + 2):
    rid = f"prefill{i}"
    engine.cache.admit(rid)
    prompt = torch.randint(0, V, (PREFILL_TOKENS,), generator=g).tolist()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    engine.runner.step([StepItem(rid, prompt, (PREFILL_TOKENS - 1,))])
    end.record()
    torch.cuda.synchronize()
    if i >= 2:
      times.append(start.elapsed_time(end))
    engine.cache.release_request(rid)
  times.sort()
  return {"ms": times[len(times) // 2]}


def kernel_table(engine, batch: int, steps: int = 6, mode: str = "decode") -> str:
  """Device time of every kernel of a decode step (a few graph replays) or of a prefill step, from CUPTI records."""
  import torch
  from torch.profiler import ProfilerActivity, profile
  from miniinfer_b200.engine import StepItem
  from miniinfer_b200.sampling import Sampler, SamplingParams
  if mode == "prefill":
    g = torch.Generator().manual_seed(7)
    V = engine.model_config.vocab_size

    def whole(i):
      rid = f"prefill{i}"
      engine.cache.admit(rid)
      engine.runner.step([StepItem(rid, torch.randint(0, V, (PREFILL_TOKENS,), generator=g).tolist(), (PREFILL_TOKENS - 1,))])
      engine.cache.release_request(rid)

    for i in range(2):
      whole(i)
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
      for i in range(steps):
        whole(10 + i)
      torch.cuda.synchronize()
    return _table_of(prof, steps, f"prefill step, {PREFILL_TOKENS} tokens")
  rids = fill_context(engine, batch, CONTEXT, seed=batch)
  params = [SamplingParams(temperature=0.6, max_tokens=GENERATED, ignore_eos=True)] * batch
  tokens_dev = torch.zeros(max(batch, 1), dtype=torch.int32, device="cuda:0")

  def one(i):
    extras = Sampler.pack(params, list(range(batch)), [i] * batch)
    engine.runner.step_and_sample([StepItem(r, [1], (0,)) for r in rids], extras, Sampler.sample, tokens_dev)

  for i in range(4):
    one(i)
  torch.cuda.synchronize()
  with profile(activities=[ProfilerActivity.CUDA]) as prof:
    for i in range(steps):
      one(10 + i)
    torch.cuda.synchronize()
  for r in rids:
    engine.cache.release_request(r)
  return _table_of(prof, steps, f"decode step, batch {batch}")


def _table_of(prof, steps: int, title: str) -> str:
  rows = []
  total = 0.0
  for ev in prof.key_averages():
    t = getattr(ev, "device_time_total", 0.0) or getattr(ev, "cuda_time_total", 0.0)
    if t <= 0:
      continue
    rows.append((t / steps, ev.count / steps, ev.key))
    total += t / steps
  rows.sort(reverse=True)
  lines = [f"{title}: {total:.1f} us of kernels per step"]
  for t, c, name in rows[:24]:
    lines.append(f"{t:9.1f} us/step  {c:6.1f} launches/step  {t / max(c, 1e-9):7.2f} us each  {name[:110]}")
  return "\n".join(lines)


def _kernel_times(fn, steps: int) -> dict:
  """Kernel name -> microseconds per step, from CUPTI records of `steps` calls of fn."""
  import torch
  from torch.profiler import ProfilerActivity, profile
  with profile(activities=[ProfilerActivity.CUDA]) as prof:
    for i in range(steps):
      fn(i)
    torch.cuda.synchronize()
  out = {}
  for ev in prof.key_averages():
    t = getattr(ev, "device_time_total", 0.0) or getattr(ev, "cuda_time_total", 0.0)
    if t > 0:
      out[ev.key] = t / steps
  return out


def _group(times: dict) -> dict:
  """Sums the kernels of a step by what they do."""
  import re
  g = {"own_products": 0.0, "library_products": 0.0, "attention": 0.0, "other": 0.0}
  for name, us in times.items():
    if "gemm_skinny" in name or "gemm_tc_kernel" in name or "gemm_stream_tc" in name:
      g["own_products"] += us
    elif re.search(r"decode_tma_kernel|decode_cluster_kernel|decode_split_kernel|decode_merge|attention_prefill", name):
      g["attention"] += us
    elif "anonymous namespace" not in name and re.search(r"nvjet|cutlass|cublas|gemm|gemv|xmma", name, re.I):
      g["library_products"] += us
    elif not name.startswith("Memcpy") and not name.startswith("Memset"):
      g["other"] += us
  return g


def kernel_rates(engine, batch: int, cfg: dict, layers: int, pk: dict, steps: int = 4) -> dict:
  """The dominant kernels of a decode step and of a prefill step with the rates they reach: the products
  stream every weight once (decode) or do the step's matrix FLOPs (prefill); the attention kernel streams
  the cache of the live requests (decode) or does the causal attention FLOPs (prefill)."""
  import torch
  from miniinfer_b200.engine import StepItem
  from miniinfer_b200.sampling import Sampler, SamplingParams
  mb = model_bytes(cfg, layers)
  rids = fill_context(engine, batch, CONTEXT, seed=1000 + batch)
  params = [SamplingParams(temperature=0.6, max_tokens=GENERATED, ignore_eos=True)] * batch
  tokens_dev = torch.zeros(max(batch, 1), dtype=torch.int32, device="cuda:0")

  def decode(i):
    extras = Sampler.pack(params, list(range(batch)), [i] * batch)
    engine.runner.step_and_sample([StepItem(r, [1], (0,)) for r in rids], extras, Sampler.sample, tokens_dev,
                                  sampling_pad=Sampler.PAD_ROWS)

  for i in range(4):
    decode(i)
  torch.cuda.synchronize()
  d = _group(_kernel_times(lambda i: decode(10 + i), steps))
  for r in rids:
    engine.cache.release_request(r)
  prod_us = d["own_products"] + d["library_products"]
  kv_bytes = batch * (CONTEXT + 4 + steps / 2.0) * mb["kv_per_token"]
  out = {"source": f"CUPTI kernel records of {steps} further steps in a process of its own, dependent launch off", "decode": {
    "products": {"us": round(prod_us, 1), "bytes": int(mb["weights"]), "GB/s": round(mb["weights"] / prod_us / 1e3, 1),
                 "frac": round(mb["weights"] / prod_us / 1e3 / pk["hbm_gbs"], 4), "own_share": round(d["own_products"] / max(prod_us, 1e-9), 3)},
    "attention": {"us": round(d["attention"], 1), "bytes": int(kv_bytes), "GB/s": round(kv_bytes / d["attention"] / 1e3, 1),
                  "frac": round(kv_bytes / d["attention"] / 1e3 / pk["hbm_gbs"], 4)},
    "other_us": round(d["other"], 1)}}

  g = torch.Generator().manual_seed(7)
  V = engine.model_config.vocab_size

  def whole(i):
    rid = f"rates{i}"
    engine.cache.admit(rid)
    engine.runner.step([StepItem(rid, torch.randint(0, V, (PREFILL_TOKENS,), generator=g).tolist(), (PREFILL_TOKENS - 1,))])
    engine.cache.release_request(rid)

  for i in range(2):
    whole(i)
  torch.cuda.synchronize()
  p = _group(_kernel_times(lambda i: whole(10 + i), 2))
  H, I, Vv = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
  nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
  T = PREFILL_TOKENS
  gemm_flops = 2.0 * T * ((nh + 2 * nkv) * hd * H + H * nh * hd + 2 * I * H + H * I) * layers + 2.0 * Vv * H
  attn_flops = layers * 2.0 * 2.0 * nh * hd * (T * (T + 1) / 2)
  prod_us = p["own_products"] + p["library_products"]
  out["prefill"] = {
    "products": {"us": round(prod_us, 1), "TFLOP": round(gemm_flops / 1e12, 4), "TFLOP/s": round(gemm_flops / prod_us / 1e6, 1),
                 "frac": round(gemm_flops / prod_us / 1e6 / pk["bf16_tflops"], 4), "own_share": round(p["own_products"] / max(prod_us, 1e-9), 3)},
    "attention": {"us": round(p["attention"], 1), "TFLOP": round(attn_flops / 1e12, 4), "TFLOP/s": round(attn_flops / p["attention"] / 1e6, 1),
                  "frac": round(attn_flops / p["attention"] / 1e6 / pk["bf16_tflops"], 4)},
    "other_us": round(p["other"], 1)}
  return out


def kernel_case(name: str, reps: int = 3) -> str:
  """One kernel alone on an input larger than L2, a few launches: the workload of the ncu summaries under
  profiles/ for the kernels that a benchmark step does not reach (or reaches only at small sizes)."""
  import torch
  from miniinfer_b200.engine.context import Workspace
  from miniinfer_b200.kernels import ops
  from miniinfer_b200.kernels.ops import AttentionBatch
  dev = torch.device("cuda:0")
  g = torch.Generator(device=dev).manual_seed(1)
  rnd = lambda *shape, dtype=torch.bfloat16, scale=1.0: (torch.randn(*shape, generator=g, device=dev) * scale).to(dtype)
  ws = Workspace(dev)

  def attention_case(dtype, page, items, **shaped):
    """items: (context length, new tokens) per request; the cache holds random keys and values.  ``shaped``: a cap on the
    scores, sigmoid weights."""
    nh, nkv, hd = 16, 8, 128
    pages_per = [-(-c // page) for c, _ in items]
    kv = rnd(sum(pages_per) + 1, 2, nkv, page, hd, dtype=dtype)
    bt = torch.zeros(len(items) + 1, max(pages_per) + 1, dtype=torch.int32)
    nxt = 1
    for b, n in enumerate(pages_per):
      bt[b, :n] = torch.arange(nxt, nxt + n)
      nxt += n
    T = sum(n for _, n in items)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    q_start, pos, tok_item, row = [], [], [], 0
    for b, (c, n) in enumerate(items):
      q_start.append(row)
      pos += list(range(c - n, c))
      tok_item += [b] * n
      row += n
    tiles = [(b, o) for b, (c, n) in enumerate(items) if n > 1 for o in range(0, n, ops.PREFILL_TILE)]
    wide = [(b, o) for b, (c, n) in enumerate(items) if n > 1 for o in range(0, n, ops.PREFILL_WIDE_TILE)]
    dec = [b for b, (c, n) in enumerate(items) if n == 1]
    batch = AttentionBatch(token_item=i32(tok_item), positions=i32(pos), seq_slot=i32(list(range(len(items)))), q_start=i32(q_start),
                           q_len=i32([n for _, n in items]), ctx_len=i32([c for c, _ in items]), num_tokens=T, num_items=len(items),
                           prefill_tiles=i32(tiles).view(-1, 2) if tiles else torch.zeros((0, 2), dtype=torch.int32, device=dev),
                           num_prefill_tiles=len(tiles), prefill_wide_tiles=i32(wide).view(-1, 2) if wide else None,
                           num_prefill_wide_tiles=len(wide), decode_items=i32(dec) if dec else torch.zeros(0, dtype=torch.int32, device=dev),
                           num_decode=len(dec), max_ctx_len=max(c for c, _ in items), scratch=ws)
    qkv = rnd(T, (nh + 2 * nkv) * hd, dtype=dtype)
    out = torch.empty(T, nh * hd, dtype=dtype, device=dev)
    if shaped.get("sigmoid"):
      shaped = {"softcap": shaped.get("softcap", 0.0), "score_bias": torch.full((nh,), -2.0, device=dev)}
    return (lambda: ops.attention(out, qkv, kv, bt.to(dev), batch, nh, nkv, hd, hd ** -0.5, None, **shaped),
            f"{len(items)} requests {items[:2]}.., page {page}, {dtype}" + (", capped scores, sigmoid weights" if shaped else ""))

  if name == "sample":
    R, V = 256, 151936
    logits = rnd(R, V, dtype=torch.float32, scale=2.0)
    f = lambda v, dt: torch.tensor(v, dtype=dt, device=dev)
    args = (f([(0.8, 1.0, 0.6, 0.0)[i % 4] for i in range(R)], torch.float32), f([(0, 50, 0, 0)[i % 4] for i in range(R)], torch.int32),
            f([(1.0, 1.0, 0.9, 1.0)[i % 4] for i in range(R)], torch.float32), f(list(range(R)), torch.int64), f([3] * R, torch.int64))
    out = torch.empty(R, dtype=torch.int32, device=dev)
    fn, what = (lambda: ops.sample(out, logits, *args, ws)), f"{R} rows x {V} float32 logits (155 MB), a quarter each: plain temperature, top-k 50, top-p 0.9, greedy"
  elif name == "silu_mul":
    gu, out = rnd(8192, 2 * 12288), torch.empty(8192, 12288, dtype=torch.bfloat16, device=dev)
    fn, what = (lambda: ops.silu_mul(out, gu)), "8192 x (2 x 12288) bf16: 403 MB in, 201 MB out"
  elif name == "gemm_f32":
    x, w = rnd(256, 4096, dtype=torch.float32), rnd(8192, 4096, dtype=torch.float32, scale=0.02)
    out = torch.empty(256, 8192, device=dev)
    fn, what = (lambda: ops.linear(out, x, w)), "float32, M = 256, N = 8192, K = 4096 (134 MB of weights, 17.2 GFLOP)"
  elif name == "gemm_tc_plain":
    x, w = rnd(2048, 4096), rnd(4096, 4096, scale=0.02)
    out = torch.empty(2048, 4096, dtype=torch.bfloat16, device=dev)
    fn, what = (lambda: ops.linear_tc(out, x, w, ws)), "bf16 plain product on tcgen05, M = 2048, N = 4096, K = 4096 (68.7 GFLOP)"
  elif name == "gemm_stream":
    x, w = rnd(8, 25600), rnd(5120, 25600, scale=0.02)
    out = torch.empty(8, 5120, dtype=torch.bfloat16, device=dev)
    fn, what = (lambda: ops.linear(out, x, w)), "bf16 few-row product on tcgen05, M = 8, N = 5120, K = 25600 (262 MB of weights: the down product of the Qwen3-32B shape)"
  elif name == "attention_generic":
    fn, what = attention_case(torch.float32, 64, [(2048, 1)] * 8 + [(2048, 512)])
  elif name == "attention_prefill_tc":
    fn, what = attention_case(torch.bfloat16, 64, [(2048, 2048)])           # the tcgen05 kernel, blocks alone
  elif name == "attention_prefill_tc_pairs":
    fn, what = attention_case(torch.bfloat16, 64, [(8192, 8192)])           # enough tiles of 128 tokens for blocks in pairs
  elif name == "attention_prefill_tc_sigmoid":
    fn, what = attention_case(torch.bfloat16, 64, [(2048, 2048)], softcap=50.0, sigmoid=True)       # the tcgen05 kernel on shaped scores
  elif name == "attention_decode_tma_sigmoid":
    fn, what = attention_case(torch.bfloat16, 64, [(2048 + 8 * i, 1) for i in range(64)], softcap=50.0, sigmoid=True)
  elif name == "attention_prefill_mma":
    fn, what = attention_case(torch.bfloat16, 16, [(2048, 2048)])           # pages of 16 tokens: not the tcgen05 kernel's
  elif name == "attention_decode_cpasync":
    fn, what = attention_case(torch.bfloat16, 16, [(2048 + 8 * i, 1) for i in range(64)])
  elif name in ("experts_many_rows", "experts_few_rows"):
    # a mixture of 32 experts (each 2 x 1536 x 4096 gate-and-up and 4096 x 1536 down: 1.2 GB in all), 8 a token:
    # 2048 tokens run the tcgen05 grouped product, 8 tokens the kernel that streams the chosen experts' weights
    T, W, F, E, top = (2048 if name == "experts_many_rows" else 8), 4096, 1536, 32, 8
    x = rnd(T, W)
    router, corr = rnd(E, W, scale=1.5 / W ** 0.5), rnd(E, dtype=torch.float32, scale=0.02)
    gate_up, down = rnd(E, 2 * F, W, scale=0.02), rnd(E, W, F, scale=0.02)
    out = torch.empty(T, W, dtype=torch.bfloat16, device=dev)
    fn = lambda: ops.routed_experts(out, x, router, corr, gate_up, down, top, ws)
    what = f"{T} tokens, {E} experts of 3 x {F} x {W}, {top} a token ({T * top * 3 * 2 * F * W / 1e9:.1f} GFLOP)"
  elif name in ("selective_scan", "delta_rule"):
    # one prompt portion of 8192 tokens (a recurrence walks it in order) beside seven decode tokens of other requests
    from types import SimpleNamespace
    cuts = [8192] + [1] * 7
    T = sum(cuts)
    it = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    ctx = SimpleNamespace(q_start=it([sum(cuts[:i]) for i in range(len(cuts))]), q_len=it(cuts), seq_slot=it(list(range(len(cuts)))),
                          num_items=len(cuts), token_item=it([b for b, n in enumerate(cuts) for _ in range(n)]))
    if name == "selective_scan":
      inner, N = 4096, 16
      u, z, dt_in, bc = rnd(T, inner), rnd(T, inner), rnd(T, inner), rnd(T, 2 * N)
      dt_b, A_log, D = rnd(inner, dtype=torch.float32) - 2.0, rnd(inner, N, dtype=torch.float32).abs(), rnd(inner, dtype=torch.float32)
      state = torch.zeros((len(cuts), inner * N), dtype=torch.float32, device=dev)
      y = torch.empty(T, inner, dtype=torch.bfloat16, device=dev)
      fn = lambda: ops.selective_scan(y, u, dt_in, bc, 0, N, z, dt_b, A_log, D, state, ctx)
      what = f"{T} tokens ({cuts[0]} of one request), {inner} channels x {N} states ({T * inner * 8 / 1e6:.0f} MB of activations in and out)"
    else:
      H, G, Dk, Dv = 16, 8, 128, 128
      q, k, v = rnd(T, G * Dk), rnd(T, G * Dk), rnd(T, H * Dv)
      a_in, b_in, gate = rnd(T, H * Dk), rnd(T, H), rnd(T, H * Dv)
      dt_bias, A_log, norm_w = rnd(H * Dk, dtype=torch.float32) - 1.0, rnd(H, dtype=torch.float32) * 0.3, 1 + 0.1 * rnd(Dv, dtype=torch.float32)
      state = torch.zeros((len(cuts), H * Dk * Dv), dtype=torch.float32, device=dev)
      out = torch.empty(T, H * Dv, dtype=torch.bfloat16, device=dev)
      fn = lambda: ops.gated_delta(out, q, k, v, a_in, b_in, gate, dt_bias, A_log, norm_w, 1e-6, state, ctx, H, G, Dk, Dv, workspace=ws)
      what = f"{T} tokens ({cuts[0]} of one request), {H} heads of {Dk} x {Dv} on {G} q/k heads"
  elif name == "linear_attention":
    # as the delta rule's case: one prompt portion of 8192 tokens beside seven decode tokens, 16 heads of 128 x 128, a decay per
    # token and key channel (the walk in order: MINIINFER_B200_LINEAR_SEGMENTS=0 in the environment; else stretches side by side)
    from types import SimpleNamespace
    cuts = [8192] + [1] * 7
    T = sum(cuts)
    it = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    ctx = SimpleNamespace(q_start=it([sum(cuts[:i]) for i in range(len(cuts))]), q_len=it(cuts), seq_slot=it(list(range(len(cuts)))),
                          num_items=len(cuts), token_item=it([b for b, n in enumerate(cuts) for _ in range(n)]),
                          positions=it([i for n in cuts for i in range(n)]))
    H, Dk, Dv = 16, 128, 128
    q, k, v, gate = rnd(T, H * Dk), rnd(T, H * Dk), rnd(T, H * Dv), rnd(T, H * Dv)
    logits, bias, norm_w = rnd(T, H * Dk, dtype=torch.float32), rnd(H * Dk, dtype=torch.float32) + 3.0, 1 + 0.1 * rnd(Dv, dtype=torch.float32)
    state = torch.zeros((len(cuts), H * Dk * Dv), dtype=torch.float32, device=dev)
    out = torch.empty(T, H * Dv, dtype=torch.bfloat16, device=dev)
    fn = lambda: ops.linear_attention(out, q, k, v, gate, state, ctx, H, Dk, Dv, 1e-6, decay_logits=logits, decay_bias=bias, tau=16.0,
                                      q_scale=Dk ** -0.5, norm_weight=norm_w, workspace=ws)
    what = f"{T} tokens ({cuts[0]} of one request), {H} heads of {Dk} x {Dv}, decays per channel"
  elif name in ("rglru_recurrence", "mingru_recurrence"):
    # one prompt portion of 8192 tokens (prepared by a kernel of its own, walked in 32 stretches a block) beside seven decode
    # tokens of other requests, 4096 channels (MINIINFER_B200_RECURRENCE_SEGMENTS=0 in the environment: the walk in order)
    from types import SimpleNamespace
    cuts = [8192] + [1] * 7
    T, C, B = sum(cuts), 4096, 8
    it = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    ctx = SimpleNamespace(q_start=it([sum(cuts[:i]) for i in range(len(cuts))]), q_len=it(cuts), seq_slot=it(list(range(len(cuts)))),
                          num_items=len(cuts), num_tokens=T, token_item=it([b for b, n in enumerate(cuts) for _ in range(n)]))
    state = torch.zeros((len(cuts), C), dtype=torch.float32, device=dev)
    out = torch.empty(T, C, dtype=torch.bfloat16, device=dev)
    if name == "rglru_recurrence":
      u, y, gates = rnd(T, C), rnd(T, C), rnd(T, 2 * C, dtype=torch.float32)
      rb, ib, yb, lam = (rnd(C, dtype=torch.float32) for _ in range(4))
      fn = lambda: ops.rglru_recurrence(out, u, gates, y, rb, ib, yb, lam - 3.0, state, ctx, B, workspace=ws)
      what = f"{T} tokens ({cuts[0]} of one request), {C} channels in {B} parts ({T * C * 14 / 1e6:.0f} MB of activations in and out)"
    else:
      proj, zb, xb = rnd(T, 3 * C), rnd(C, dtype=torch.float32), rnd(C, dtype=torch.float32)
      fn = lambda: ops.mingru_recurrence(out, proj, zb, xb, state, ctx, workspace=ws)
      what = f"{T} tokens ({cuts[0]} of one request), {C} channels ({T * C * 8 / 1e6:.0f} MB of activations in and out)"
  elif name == "hyper_connection":
    # the kernel between two sublayers: 16384 rows of 4 streams x 2048 values float32 (537 MB, read and written) and a bfloat16 sublayer output
    T, S, W = 16384, 4, 2048
    streams, y = rnd(T, S * W, dtype=torch.float32), rnd(T, W)
    mix, out_w, in_w = torch.eye(S, device=dev) + 0.1 * rnd(S, S, dtype=torch.float32), rnd(S, dtype=torch.float32), rnd(S, dtype=torch.float32)
    norm_w = 1 + 0.1 * rnd(W, dtype=torch.float32)
    res = torch.empty(T, W, dtype=torch.bfloat16, device=dev)
    fn = lambda: ops.hyper_connection(res, streams, y, mix, out_w, in_w, norm_w, 1e-6)
    what = f"{T} rows of {S} streams x {W} float32 ({(2 * T * S * W * 4 + 2 * T * W * 2) / 1e6:.0f} MB in and out)"
  else:
    raise SystemExit(f"unknown kernel case {name!r}")
  fn()
  torch.cuda.synchronize()
  start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  start.record()
  for _ in range(reps):
    fn()
  end.record()
  torch.cuda.synchronize()
  return f"{name}: {what}: {1000 * start.elapsed_time(end) / reps:.1f} us per call (warm, {reps} calls back to back)"


KERNEL_CASES = ("sample", "silu_mul", "gemm_f32", "gemm_tc_plain", "gemm_stream", "attention_generic", "attention_prefill_tc",
                "attention_prefill_tc_pairs", "attention_prefill_mma", "attention_decode_cpasync", "experts_many_rows", "experts_few_rows",
                "selective_scan", "delta_rule", "linear_attention", "hyper_connection", "attention_prefill_tc_sigmoid", "attention_decode_tma_sigmoid",
                "rglru_recurrence", "mingru_recurrence")


def mixed_workload(model_dir: str, requests: int = 64, outputs: int = 256) -> dict:
  """A continuous batch through `LLMEngine.generate`: prompts of 128 .. 2048 uniform random tokens, `outputs`
  generated tokens each, prompts cut under a budget of 2048 tokens a step.  Run twice; the second run
  (graphs recorded, kernels loaded) is reported."""
  import torch
  from miniinfer_b200 import LLMEngine, SamplingParams
  pages = requests * (-(-(2048 + outputs) // PAGE) + 1) + 8
  engine = LLMEngine(model_dir, dtype="bfloat16", device="cuda:0", load_format="random", page_size=PAGE, num_pages=pages,
                     max_num_seqs=requests, max_model_len=MAX_MODEL_LEN, max_num_batched_tokens=PREFILL_TOKENS, seed=0)
  g = torch.Generator().manual_seed(0)
  lens = torch.randint(128, 2049, (requests,), generator=g).tolist()
  V = engine.model_config.vocab_size
  prompts = [torch.randint(0, V, (n,), generator=g).tolist() for n in lens]
  sp = SamplingParams(temperature=0.6, max_tokens=outputs, ignore_eos=True)
  res = {}
  for _ in range(2):
    s0 = dict(engine.stats)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    engine.generate(prompts, sp)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    steps = engine.stats["steps"] - s0["steps"]
    res = {"workload": f"{requests} requests, prompts 128..2048, {outputs} outputs each, 2048 tokens a step",
           "seconds": round(dt, 3), "prompt_tokens": sum(lens), "output_tokens": requests * outputs,
           "total_tok_s": round((sum(lens) + requests * outputs) / dt, 1), "output_tok_s": round(requests * outputs / dt, 1),
           "steps": steps, "ms_per_step": round(1000 * dt / steps, 3)}
  return res


REF_DIR = os.path.join(ROOT, "baseline", "_ref")


def _write_reference_model(cfg: dict, out_dir: str, seed: int = 0) -> None:
  """A model folder the reference can load, made without this repository's package: config.json,
  model.safetensors with the tensor names of the Qwen3 checkpoints (random N(0, 0.02) matrices, norm
  weights near one) and a word-level tokenizer of the configuration's vocabulary size."""
  import torch
  from safetensors.torch import save_file
  from tokenizers import Tokenizer, models, pre_tokenizers
  os.makedirs(out_dir, exist_ok=True)
  with open(os.path.join(out_dir, "config.json"), "w") as f:
    json.dump(dict(cfg, torch_dtype="bfloat16", hidden_act="silu", attention_bias=False, use_sliding_window=False,
                   bos_token_id=0, eos_token_id=1), f)
  g = torch.Generator().manual_seed(seed)
  H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
  nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
  mat = lambda *s: (torch.randn(*s, generator=g) * 0.02).to(torch.bfloat16)
  vec = lambda n: (1 + 0.1 * torch.randn(n, generator=g)).to(torch.bfloat16)
  sd = {"model.embed_tokens.weight": mat(V, H), "model.norm.weight": vec(H)}
  for i in range(cfg["num_hidden_layers"]):
    p = f"model.layers.{i}"
    sd.update({f"{p}.input_layernorm.weight": vec(H), f"{p}.post_attention_layernorm.weight": vec(H),
               f"{p}.self_attn.q_proj.weight": mat(nh * hd, H), f"{p}.self_attn.k_proj.weight": mat(nkv * hd, H),
               f"{p}.self_attn.v_proj.weight": mat(nkv * hd, H), f"{p}.self_attn.o_proj.weight": mat(H, nh * hd),
               f"{p}.self_attn.q_norm.weight": vec(hd), f"{p}.self_attn.k_norm.weight": vec(hd),
               f"{p}.mlp.gate_proj.weight": mat(I, H), f"{p}.mlp.up_proj.weight": mat(I, H), f"{p}.mlp.down_proj.weight": mat(H, I)})
  if not cfg.get("tie_word_embeddings"):
    sd["lm_head.weight"] = mat(V, H)
  save_file(sd, os.path.join(out_dir, "model.safetensors"))
  vocab = {"<bos>": 0, "<eos>": 1, "<unk>": 2}
  for i in range(3, V):
    vocab[f"t{i}"] = i
  tok = Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
  tok.pre_tokenizer = pre_tokenizers.Whitespace()
  tok.save(os.path.join(out_dir, "tokenizer.json"))
  with open(os.path.join(out_dir, "tokenizer_config.json"), "w") as f:
    json.dump({"tokenizer_class": "PreTrainedTokenizerFast", "bos_token": "<bos>", "eos_token": "<eos>", "unk_token": "<unk>",
               "pad_token": "<eos>", "model_max_length": cfg["max_position_embeddings"]}, f)


def reference_child(args) -> int:
  """Runs in a process of its own, with nothing of this repository's package imported: the reference as
  installed under baseline/_ref (its sub-packages lie there at top level, so the name ``miniinfer`` is
  bound to that folder), its own ``LLMEngine.generate`` with token-id prompts, as its benchmark does
  (benchmark/bench_miniinfer.py:28-58).  Decode tokens a second: two runs that differ only in the number
  of generated tokens, (tokens of the longer - tokens of the shorter) / (time of the longer - the shorter)."""
  import types
  pkg = types.ModuleType("miniinfer")
  pkg.__path__ = [REF_DIR]
  sys.modules["miniinfer"] = pkg
  sys.path.insert(0, REF_DIR)
  os.environ.update(HF_HUB_OFFLINE="1", TRANSFORMERS_OFFLINE="1")
  import torch
  from miniinfer.engine.llm_engine import LLMEngine
  from miniinfer.utils.sampling_params import SamplingParams
  cfg = dict(MODEL, **SHAPES[args.shape])
  if args.layers:
    cfg["num_hidden_layers"] = args.layers
  context = args.context if args.context is not None else SHAPE_CONTEXT.get(args.shape, CONTEXT)
  steps, warmup, batch = args.steps, max(args.warmup, 3), args.batch
  with tempfile.TemporaryDirectory() as d:
    _write_reference_model(cfg, d)
    # no dtype is passed: the reference's engine builds its model in float16 whatever it is asked for
    # (miniinfer/engine/model_runner.py:66-68, models/fused_qwen3.py:272), and its cache must match
    engine = LLMEngine(model=d, use_multiprocess=False, max_num_seqs=max(batch, 8),
                       max_context_len=max(MAX_MODEL_LEN, SHAPE_MAX_MODEL_LEN.get(args.shape, 0)), page_size=PAGE * 4,
                       enable_prefix_cache=False, debug=False)
    engine.start()
    g = torch.Generator().manual_seed(1)
    V = cfg["vocab_size"]

    def run(n_tokens: int) -> float:
      prompts = [torch.randint(3, V, (context,), generator=g).tolist() for _ in range(batch)]
      sp = SamplingParams(temperature=0.6, ignore_eos=True, max_tokens=n_tokens)
      torch.cuda.synchronize()
      t0 = time.perf_counter()
      outs = engine.generate(prompts=prompts, sampling_params=sp, use_tqdm=False)
      torch.cuda.synchronize()
      dt = time.perf_counter() - t0
      assert all(len(o["token_ids"]) == n_tokens for o in outs), "the reference generated another number of tokens"
      return dt

    run(warmup + 4)                      # loads kernels, records its CUDA graphs
    clocks = ClockSampler()
    clocks.start()
    short = min(run(4) for _ in range(2))
    long_ = min(run(4 + steps) for _ in range(2))
    clock_info = clocks.stop()
    engine.stop()
  ms = 1000.0 * (long_ - short) / steps
  value = batch * 1000.0 / ms
  print(json.dumps({
    "metric": f"decode tok/s at batch {batch} (Qwen3-{args.shape.upper()} shape, {context}-token contexts)",
    "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": round(ms, 4),
    "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp16 (the reference's own; same width as bf16)", "impl": "reference",
    "data": "synthetic: random weights N(0, 0.02), uniform random token ids",
    "config": {"model": f"Qwen3-{args.shape.upper()} shape", "layers": cfg["num_hidden_layers"], "global_batch": batch, "seq_len": context,
               "page_size": PAGE * 4, "attention_backend": "the reference's default", "parallelism": "single GPU",
               "timing": "LLMEngine.generate end to end, host tokens in and out; (time of 4+K tokens - time of 4 tokens) / K"},
    "e2e": {"value": round(value, 1), "unit": "tok/s", "ms_per_step": round(ms, 4)},
    "clocks": clock_info}))
  return 0


def reference_arm(args) -> int:
  """The reference's own engine on the same shape, batch, context and step count, in a child process.
  If it cannot be imported or run, one line says which import or call failed."""
  if not os.path.isdir(REF_DIR):
    print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref does not exist: the reference was not installed here"}))
    return 0
  cmd = [sys.executable, os.path.abspath(__file__), "--impl", "reference-child", "--steps", str(args.steps), "--warmup", str(args.warmup),
         "--batch", str(args.batch), "--shape", args.shape]
  if args.layers:
    cmd += ["--layers", str(args.layers)]
  if args.context is not None:
    cmd += ["--context", str(args.context)]
  try:
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=1500)
  except subprocess.TimeoutExpired:
    print(json.dumps({"impl": "reference", "unavailable": "the reference's engine did not finish within 25 minutes"}))
    return 0
  lines = [l for l in proc.stdout.splitlines() if l.startswith("{") and '"impl": "reference"' in l]
  if proc.returncode == 0 and lines:
    print(lines[-1])
    return 0
  err = [l.strip() for l in (proc.stderr or "").splitlines() if l.strip()]
  why = err[-1] if err else f"exit code {proc.returncode} without a message"
  where = next((l for l in reversed(err) if l.startswith("File ") and "_ref" in l), "")
  print(json.dumps({"impl": "reference", "unavailable": f"the reference's own code failed: {why[:300]} {where[:200]}".strip()}))
  return 0


# ---------------------------------------------------------------------------------------------- --compare rikanex
# Sizes for the comparison of the Rikanex design with the Qwen3 dense decoder at equal size: width, query / kv heads, head
# size, the dense feed-forward's width, and the experts that stand for it (count, width, per token) so that a token
# passes through as many feed-forward weights in both; layers; both models get the same sliding window and vocabulary.
COMPARE_SIZES = {
  "s": dict(width=1024, heads=16, kv_heads=8, head=128, ff=3072, experts=8, expert_ff=768, top=4, layers=8),
  "m": dict(width=2048, heads=32, kv_heads=8, head=64, ff=6144, experts=16, expert_ff=1536, top=4, layers=6),
  "l": dict(width=4096, heads=32, kv_heads=8, head=128, ff=12288, experts=32, expert_ff=1536, top=8, layers=4),
}
COMPARE_WINDOW = 1024
COMPARE_VOCAB = 32768


def compare_configs(size: dict) -> dict:
  W, H, G, hd = size["width"], size["heads"], size["kv_heads"], size["head"]
  qwen = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=size["layers"], hidden_size=W,
              num_attention_heads=H, num_key_value_heads=G, head_dim=hd, intermediate_size=size["ff"], vocab_size=COMPARE_VOCAB,
              rope_theta=1000000.0, rms_norm_eps=1e-6, max_position_embeddings=40960, tie_word_embeddings=False,
              use_sliding_window=True, sliding_window=COMPARE_WINDOW, max_window_layers=0)
  mixer = {"heads": H, "kv_heads": G, "dim": hd, "vdim": hd, "scale": hd ** -0.5, "mask": {"size": COMPARE_WINDOW}, "v_mix": True}
  moe = {"kind": "moe", "expert": {"ff": size["expert_ff"]}, "router": {"experts": size["experts"], "top": size["top"]}}
  layers = [{"type": "attention", "mixer": dict(mixer), "mlp": {"kind": "dense", "ff": size["ff"]} if i == 0 else moe}
            for i in range(size["layers"])]
  rikanex = {"architecture": "Rikanex", "vocab": COMPARE_VOCAB, "width": W, "embedding": {"scale": 8.0}, "norm": {"eps": 1e-6},
             "layers": layers}
  return {"qwen3": qwen, "rikanex": rikanex}


def _compare_groups(times: dict) -> dict:
  import re
  g = {"attention": 0.0, "experts": 0.0, "dense_products": 0.0, "routing": 0.0, "other": 0.0}
  for name, us in times.items():
    if re.search(r"decode_tma_kernel|decode_cluster_kernel|decode_split_kernel|decode_merge|attention_prefill|attention_generic", name):
      g["attention"] += us
    elif "moe_gemm" in name or "moe_stream" in name or re.search(r"gemm_tc_kernel<\w+, \w+, (true|\(bool\)1)[,>]", name):     # the grouped instantiation of the tcgen05 product
      g["experts"] += us
    elif re.search(r"moe_route|moe_align|moe_combine", name):
      g["routing"] += us
    elif "gemm_skinny" in name or "gemm_tc_kernel" in name or "gemm_stream_tc" in name or \
        ("anonymous namespace" not in name and re.search(r"nvjet|cutlass|cublas|gemm|gemv|xmma", name, re.I)):
      g["dense_products"] += us
    elif not name.startswith("Memcpy") and not name.startswith("Memset"):
      g["other"] += us
  return g


def compare_one(name: str, cfg: dict, size: dict, batch: int, steps: int, warmup: int, pk: dict, kernels: bool) -> dict:
  """Prefill and decode of one model of the comparison; with ``kernels`` the device time of its kinds of kernels and the
  rates they reach against the measured peaks (run with dependent launch off, see main)."""
  import torch
  from miniinfer_b200.engine import StepItem
  from miniinfer_b200.sampling import Sampler, SamplingParams
  W, H, G, hd, L = size["width"], size["heads"], size["kv_heads"], size["head"], size["layers"]
  win, T = COMPARE_WINDOW, PREFILL_TOKENS
  with tempfile.TemporaryDirectory() as d:
    with open(os.path.join(d, "config.json"), "w") as f:
      json.dump(cfg, f)
    engine = build_engine(d, batch)
    out = {}
    if not kernels:
      dec = time_decode(engine, batch, steps, warmup)
      pre = time_prefill(engine)
      out = {"decode_tok_s": round(dec["tok_s"], 1), "decode_ms": round(dec["ms"], 4), "launches_per_decode_step": int(dec["launches_per_step"]),
             "prefill_tok_s": round(T / (pre["ms"] * 1e-3), 1), "prefill_ms": round(pre["ms"], 3)}
    else:
      rids = fill_context(engine, batch, CONTEXT, seed=1000 + batch)
      params = [SamplingParams(temperature=0.6, max_tokens=GENERATED, ignore_eos=True)] * batch
      tokens_dev = torch.zeros(max(batch, 1), dtype=torch.int32, device="cuda:0")

      def decode(i):
        extras = Sampler.pack(params, list(range(batch)), [i] * batch)
        engine.runner.step_and_sample([StepItem(r, [1], (0,)) for r in rids], extras, Sampler.sample, tokens_dev,
                                      sampling_pad=Sampler.PAD_ROWS)

      for i in range(4):
        decode(i)
      torch.cuda.synchronize()
      dk = _compare_groups(_kernel_times(lambda i: decode(10 + i), 4))
      for r in rids:
        engine.cache.release_request(r)
      g = torch.Generator().manual_seed(7)

      def whole(i):
        rid = f"rates{i}"
        engine.cache.admit(rid)
        engine.runner.step([StepItem(rid, torch.randint(0, COMPARE_VOCAB, (T,), generator=g).tolist(), (T - 1,))])
        engine.cache.release_request(rid)

      for i in range(2):
        whole(i)
      torch.cuda.synchronize()
      pk_times = _compare_groups(_kernel_times(lambda i: whole(10 + i), 2))
      # what each kind of kernel has to do
      seen = sum(min(t + 1, win) for t in range(T))
      attn_flops = L * 4.0 * H * hd * seen
      attn_bytes = batch * min(CONTEXT, win) * L * 2 * G * hd * 2
      moe_layers = L - 1 if name == "rikanex" else 0
      E, F, top = size["experts"], size["expert_ff"], size["top"]
      touched = E * (1.0 - (1.0 - top / E) ** batch)             # experts a decode step of `batch` tokens reads if choices are uniform
      if name == "rikanex":
        # what the last step's last routed layer did read: the row tiles that an expert owns (few rows: a tile an expert)
        for gph in engine.runner._graphs.values():
          buf = gph.ws._bufs.get(("moe_tile_expert", torch.int32))
          if buf is not None:
            touched = float((buf >= 0).sum().item())
      for grp in (pk_times, dk):
        for key in grp:
          grp[key] = max(grp[key], 1e-9)
      rates = {"prefill_attention": {"us": round(pk_times["attention"], 1), "TFLOP/s": round(attn_flops / pk_times["attention"] / 1e6, 1),
                                     "frac": round(attn_flops / pk_times["attention"] / 1e6 / pk["bf16_tflops"], 4)},
               "decode_attention": {"us": round(dk["attention"], 1), "GB/s": round(attn_bytes / dk["attention"] / 1e3, 1),
                                    "frac": round(attn_bytes / dk["attention"] / 1e3 / pk["hbm_gbs"], 4)}}
      if moe_layers:
        moe_flops = moe_layers * T * top * 3 * 2.0 * F * W
        moe_bytes = moe_layers * touched * 3 * F * W * 2
        rates["prefill_experts"] = {"us": round(pk_times["experts"], 1), "TFLOP/s": round(moe_flops / pk_times["experts"] / 1e6, 1),
                                    "frac": round(moe_flops / pk_times["experts"] / 1e6 / pk["bf16_tflops"], 4)}
        rates["decode_experts"] = {"us": round(dk["experts"], 1), "GB/s": round(moe_bytes / dk["experts"] / 1e3, 1),
                                   "frac": round(moe_bytes / dk["experts"] / 1e3 / pk["hbm_gbs"], 4)}
        rates["decode_experts"]["experts_read_per_layer"] = round(touched, 1)
        rates["routing_us"] = {"prefill": round(pk_times["routing"], 1), "decode": round(dk["routing"], 1)}
      dense_ff = (L - moe_layers) * 3 * size["ff"] * W
      proj = L * ((H + 2 * G) * hd * W + W * H * hd + (H * hd * W if name == "rikanex" else 0))
      dense_w = dense_ff + proj + COMPARE_VOCAB * W
      rates["prefill_dense_products"] = {"us": round(pk_times["dense_products"], 1),
                                         "TFLOP/s": round(2.0 * T * (dense_ff + proj) / pk_times["dense_products"] / 1e6, 1),
                                         "frac": round(2.0 * T * (dense_ff + proj) / pk_times["dense_products"] / 1e6 / pk["bf16_tflops"], 4)}
      rates["decode_dense_products"] = {"us": round(dk["dense_products"], 1), "GB/s": round(2.0 * dense_w / dk["dense_products"] / 1e3, 1),
                                        "frac": round(2.0 * dense_w / dk["dense_products"] / 1e3 / pk["hbm_gbs"], 4)}
      rates["other_us"] = {"prefill": round(pk_times["other"], 1), "decode": round(dk["other"], 1)}
      out = rates
    engine.stop()
    del engine
    gc.collect()
    torch.cuda.empty_cache()
  return out


# ---------------------------------------------------------------------------------------------- --compare vugudra
# Sizes for the comparison of the Vugudra design with the Qwen3 dense decoder at equal size: width, dense feed-forward,
# layers, and the sizes of the three mixers at about the weights of the dense decoder's attention.  The layers go
# selective scan, latent attention, windowed attention beside a gated delta rule, and again; the Qwen3 model has the heads
# of the windowed attention, its window and the same vocabulary.
VUGUDRA_SIZES = {
  "s": dict(width=1024, ff=3072, layers=6, heads=16, kv_heads=8, head=128,
            scan=dict(inner=2048, state=16, dt_rank=64, conv=4),
            latent=dict(heads=16, dim=64, rot_dim=32, vdim=64, kv_rank=192, q_rank=384),
            delta=dict(heads=8, kv_heads=4, dim=128, vdim=128, conv=4, rank=64)),
  "m": dict(width=2048, ff=6144, layers=6, heads=32, kv_heads=8, head=64,
            scan=dict(inner=4096, state=16, dt_rank=128, conv=4),
            latent=dict(heads=32, dim=64, rot_dim=64, vdim=64, kv_rank=192, q_rank=768),
            delta=dict(heads=16, kv_heads=8, dim=128, vdim=128, conv=4, rank=128)),
  "l": dict(width=4096, ff=12288, layers=3, heads=32, kv_heads=8, head=128,
            scan=dict(inner=8192, state=16, dt_rank=256, conv=4),
            latent=dict(heads=32, dim=128, rot_dim=64, vdim=128, kv_rank=192, q_rank=1536),
            delta=dict(heads=32, kv_heads=16, dim=128, vdim=128, conv=4, rank=128)),
}
VUGUDRA_KEEP_FIRST = 4


def vugudra_configs(size: dict) -> dict:
  W, H, G, hd, L = size["width"], size["heads"], size["kv_heads"], size["head"], size["layers"]
  qwen = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=L, hidden_size=W,
              num_attention_heads=H, num_key_value_heads=G, head_dim=hd, intermediate_size=size["ff"], vocab_size=COMPARE_VOCAB,
              rope_theta=1000000.0, rms_norm_eps=1e-6, max_position_embeddings=40960, tie_word_embeddings=False,
              use_sliding_window=True, sliding_window=COMPARE_WINDOW, max_window_layers=0)
  mlp = {"kind": "dense", "ff": size["ff"]}
  lat, dl = size["latent"], size["delta"]
  kinds = [
    {"type": "mamba1", "mixer": dict(size["scan"]), "mlp": mlp},
    {"type": "latent_attention", "mlp": mlp,
     "mixer": dict({k: lat[k] for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank")}, scale=(lat["dim"] + lat["rot_dim"]) ** -0.5,
                   rot={"dims": lat["rot_dim"], "base": 10000.0, "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}})},
    {"type": "parallel", "mlp": mlp,
     "mixer": {"left": {"heads": H, "kv_heads": G, "dim": hd, "vdim": hd, "scale": hd ** -0.5, "rot": {"dims": hd, "base": 1000000.0},
                        "mask": {"size": COMPARE_WINDOW, "keep_first": VUGUDRA_KEEP_FIRST}},
               "right": {k: dl[k] for k in ("heads", "kv_heads", "dim", "vdim", "conv")}}},
  ]
  layers = [kinds[i % 3] for i in range(L)]
  ranks = {f"l{i}.{w}": dl["rank"] for i in range(L) if i % 3 == 2 for w in ("decay", "gate")}
  vug = {"architecture": "Vugudra", "vocab": COMPARE_VOCAB, "width": W, "norm": {"eps": 1e-6}, "layers": layers, "low_ranks": ranks}
  return {"qwen3": qwen, "vugudra": vug}


def _vugudra_groups(times: dict) -> dict:
  import re
  g = {"attention": 0.0, "dense_products": 0.0, "head_products": 0.0, "scan": 0.0, "delta_rule": 0.0, "convolution": 0.0, "other": 0.0}
  for name, us in times.items():
    if re.search(r"decode_tma_kernel|decode_cluster_kernel|decode_split_kernel|decode_merge|attention_prefill|attention_generic", name):
      g["attention"] += us
    elif "gemm_batched" in name:
      g["head_products"] += us
    elif "selective_scan" in name or "scan_carry" in name:
      g["scan"] += us
    elif "gated_delta" in name or "delta_recurrence" in name or "delta_prepare" in name or "delta_output" in name or "delta_carry" in name:
      g["delta_rule"] += us
    elif "causal_conv" in name or "conv_state" in name:
      g["convolution"] += us
    elif "gemm_skinny" in name or "gemm_tc_kernel" in name or "gemm_stream_tc" in name or \
        ("anonymous namespace" not in name and re.search(r"nvjet|cutlass|cublas|gemm|gemv|xmma", name, re.I)):
      g["dense_products"] += us
    elif not name.startswith("Memcpy") and not name.startswith("Memset"):
      g["other"] += us
  return g


def vugudra_one(name: str, cfg: dict, size: dict, batch: int, steps: int, warmup: int, pk: dict, kernels: bool) -> dict:
  """Prefill and decode of one model of the comparison; with ``kernels`` the device time of its kinds of kernels and the
  rates they reach against the measured peaks (run with dependent launch off, see main)."""
  import torch
  from miniinfer_b200.engine import StepItem
  from miniinfer_b200.sampling import Sampler, SamplingParams
  W, H, G, hd, L = size["width"], size["heads"], size["kv_heads"], size["head"], size["layers"]
  win, T = COMPARE_WINDOW, PREFILL_TOKENS
  with tempfile.TemporaryDirectory() as d:
    with open(os.path.join(d, "config.json"), "w") as f:
      json.dump(cfg, f)
    engine = build_engine(d, batch)
    if not kernels:
      dec = time_decode(engine, batch, steps, warmup)
      pre = time_prefill(engine)
      out = {"decode_tok_s": round(dec["tok_s"], 1), "decode_ms": round(dec["ms"], 4), "launches_per_decode_step": int(dec["launches_per_step"]),
             "prefill_tok_s": round(T / (pre["ms"] * 1e-3), 1), "prefill_ms": round(pre["ms"], 3)}
    else:
      rids = fill_context(engine, batch, CONTEXT, seed=1000 + batch)
      params = [SamplingParams(temperature=0.6, max_tokens=GENERATED, ignore_eos=True)] * batch
      tokens_dev = torch.zeros(max(batch, 1), dtype=torch.int32, device="cuda:0")

      def decode(i):
        extras = Sampler.pack(params, list(range(batch)), [i] * batch)
        engine.runner.step_and_sample([StepItem(r, [1], (0,)) for r in rids], extras, Sampler.sample, tokens_dev,
                                      sampling_pad=Sampler.PAD_ROWS)

      for i in range(4):
        decode(i)
      torch.cuda.synchronize()
      dtimes = _kernel_times(lambda i: decode(10 + i), 4)
      dk = _vugudra_groups(dtimes)
      for r in rids:
        engine.cache.release_request(r)
      g = torch.Generator().manual_seed(7)

      def whole(i):
        rid = f"rates{i}"
        engine.cache.admit(rid)
        engine.runner.step([StepItem(rid, torch.randint(0, COMPARE_VOCAB, (T,), generator=g).tolist(), (T - 1,))])
        engine.cache.release_request(rid)

      for i in range(2):
        whole(i)
      torch.cuda.synchronize()
      ptimes = _kernel_times(lambda i: whole(10 + i), 2)
      pt = _vugudra_groups(ptimes)
      for grp in (pt, dk):
        for key in grp:
          grp[key] = max(grp[key], 1e-9)
      ff_w = L * 3 * size["ff"] * W
      if name == "qwen3":
        seen = sum(min(t + 1, win) for t in range(T))
        attn_flops = L * 4.0 * H * hd * seen
        attn_bytes = batch * min(CONTEXT, win) * L * 2 * G * hd * 2
        proj_w = L * ((H + 2 * G) * hd * W + W * H * hd)
        extra = {}
      else:
        sc, lat, dl = size["scan"], size["latent"], size["delta"]
        n_scan, n_lat, n_side = (L + 2) // 3, (L + 1) // 3, L // 3
        lat_hd = lat["kv_rank"] + lat["rot_dim"]
        seen_win = sum(min(t + 1, win + VUGUDRA_KEEP_FIRST) for t in range(T))
        seen_all = sum(t + 1 for t in range(T))
        # scores over the keys a token sees, and the weighted values: latent heads read kv_rank + rot_dim and give kv_rank
        attn_flops = n_side * 4.0 * H * hd * seen_win + n_lat * 2.0 * lat["heads"] * (lat_hd + lat["kv_rank"]) * seen_all
        lat_row = -(-lat_hd // 16) * 16
        attn_bytes = batch * 2 * (n_side * min(CONTEXT, win + VUGUDRA_KEEP_FIRST) * 2 * G * hd + n_lat * CONTEXT * 2 * lat_row)
        I, N, R = sc["inner"], sc["state"], sc["dt_rank"]
        scan_w = 2 * I * W + (R + 2 * N) * I + I * R + W * I
        lat_w = (lat["q_rank"] + lat["kv_rank"] + lat["rot_dim"] + lat["heads"]) * W + lat["heads"] * (lat["dim"] + lat["rot_dim"]) * lat["q_rank"] + W * lat["heads"] * lat["vdim"]
        left_w = (H + G) * hd * W + W * H * hd
        dh, dg, dd, dv, rk = dl["heads"], dl["kv_heads"], dl["dim"], dl["vdim"], dl["rank"]
        right_w = (2 * dg * dd + dh * dv + dh + 2 * rk) * W + rk * (dh * dd + dh * dv) + W * dh * dv
        proj_w = n_scan * scan_w + n_lat * lat_w + n_side * (left_w + right_w)
        head_w = n_lat * lat["heads"] * lat["kv_rank"] * (lat["dim"] + lat["vdim"])
        # what the recurrences must move: their inputs and outputs once (2 bytes a value) and, in a decode step, every
        # request's state in and out (4 bytes a value)
        scan_io = n_scan * (4 * I + 2 * N) * 2
        scan_state = n_scan * I * N * 4 * 2
        delta_io = n_side * (2 * dg * dd + dh * (3 * dv + dd + 1)) * 2
        delta_state = n_side * dh * dd * dv * 4 * 2
        extra = {
          "prefill_head_products": {"us": round(pt["head_products"], 1), "TFLOP/s": round(2.0 * T * head_w / pt["head_products"] / 1e6, 1),
                                    "frac": round(2.0 * T * head_w / pt["head_products"] / 1e6 / pk["bf16_tflops"], 4)},
          "decode_head_products": {"us": round(dk["head_products"], 1), "GB/s": round(2.0 * head_w / dk["head_products"] / 1e3, 1),
                                   "frac": round(2.0 * head_w / dk["head_products"] / 1e3 / pk["hbm_gbs"], 4)},
          "prefill_scan": {"us": round(pt["scan"], 1), "GB/s": round(T * scan_io / pt["scan"] / 1e3, 1),
                           "frac": round(T * scan_io / pt["scan"] / 1e3 / pk["hbm_gbs"], 4)},
          "decode_scan": {"us": round(dk["scan"], 1), "GB/s": round(batch * (scan_io + scan_state) / dk["scan"] / 1e3, 1),
                          "frac": round(batch * (scan_io + scan_state) / dk["scan"] / 1e3 / pk["hbm_gbs"], 4)},
          "prefill_delta_rule": {"us": round(pt["delta_rule"], 1), "GB/s": round(T * delta_io / pt["delta_rule"] / 1e3, 1),
                                 "frac": round(T * delta_io / pt["delta_rule"] / 1e3 / pk["hbm_gbs"], 4)},
          "decode_delta_rule": {"us": round(dk["delta_rule"], 1), "GB/s": round(batch * (delta_io + delta_state) / dk["delta_rule"] / 1e3, 1),
                                "frac": round(batch * (delta_io + delta_state) / dk["delta_rule"] / 1e3 / pk["hbm_gbs"], 4)},
          "convolution_us": {"prefill": round(pt["convolution"], 1), "decode": round(dk["convolution"], 1)},
        }
      dense_w = ff_w + proj_w + COMPARE_VOCAB * W
      out = {"prefill_attention": {"us": round(pt["attention"], 1), "TFLOP/s": round(attn_flops / pt["attention"] / 1e6, 1),
                                   "frac": round(attn_flops / pt["attention"] / 1e6 / pk["bf16_tflops"], 4)},
             "decode_attention": {"us": round(dk["attention"], 1), "GB/s": round(attn_bytes / dk["attention"] / 1e3, 1),
                                  "frac": round(attn_bytes / dk["attention"] / 1e3 / pk["hbm_gbs"], 4)},
             "prefill_dense_products": {"us": round(pt["dense_products"], 1),
                                        "TFLOP/s": round(2.0 * T * (ff_w + proj_w) / pt["dense_products"] / 1e6, 1),
                                        "frac": round(2.0 * T * (ff_w + proj_w) / pt["dense_products"] / 1e6 / pk["bf16_tflops"], 4)},
             "decode_dense_products": {"us": round(dk["dense_products"], 1), "GB/s": round(2.0 * dense_w / dk["dense_products"] / 1e3, 1),
                                       "frac": round(2.0 * dense_w / dk["dense_products"] / 1e3 / pk["hbm_gbs"], 4)},
             "other_us": {"prefill": round(pt["other"], 1), "decode": round(dk["other"], 1)}}
      out.update(extra)

      def top(times):
        rows = sorted(((us, n) for n, us in times.items() if not n.startswith("Mem")), reverse=True)[:14]
        return [[round(us, 1), n.replace("(anonymous namespace)::", "")[:70]] for us, n in rows]

      out["top_kernels_us"] = {"prefill": top(ptimes), "decode": top(dtimes)}
    engine.stop()
    del engine
    gc.collect()
    torch.cuda.empty_cache()
  return out


# ---------------------------------------------------------------------------------------------- --compare famupel
# Sizes for the comparison of the Famupel design with the closest design the engine has, Vugudra (attention beside a
# recurrence with a matrix state a head, recurrent layers between), at equal size: the sizes of the Vugudra comparison and,
# for Famupel, gated linear attention and retention with the delta rule's heads and state (128 x 128 a head), the
# attention's heads without a window, a feed-forward of two matrices with the weights of the gated one's three, and
# residual streams.  The layers go gated linear attention twice, attention beside retention, and again.
FAMUPEL_SIZES = {
  "s": dict(VUGUDRA_SIZES["s"], gla=dict(heads=8, dim=128, vdim=128, rank=64, tau=16.0), ret=dict(heads=8, dim=128, vdim=128), streams=2),
  "m": dict(VUGUDRA_SIZES["m"], gla=dict(heads=16, dim=128, vdim=128, rank=128, tau=16.0), ret=dict(heads=16, dim=128, vdim=128), streams=2),
  "l": dict(VUGUDRA_SIZES["l"], gla=dict(heads=32, dim=128, vdim=128, rank=128, tau=16.0), ret=dict(heads=32, dim=128, vdim=128), streams=4),
}


def famupel_configs(size: dict) -> dict:
  W, H, G, hd, L = size["width"], size["heads"], size["kv_heads"], size["head"], size["layers"]
  gl, rt = size["gla"], size["ret"]
  mlp = {"kind": "dense", "ff": size["ff"] * 3 // 2}
  kinds = [
    {"type": "gla", "mixer": {k: gl[k] for k in ("heads", "dim", "vdim", "tau")}, "mlp": mlp},
    {"type": "gla", "mixer": {k: gl[k] for k in ("heads", "dim", "vdim", "tau")}, "mlp": mlp},
    {"type": "parallel", "mlp": mlp,
     "mixer": {"left": {"heads": H, "kv_heads": G, "dim": hd, "vdim": hd, "scale": hd ** -0.5,
                        "rot": {"dims": hd, "base": 500000.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}},
               "right": {"heads": rt["heads"], "dim": rt["dim"], "vdim": rt["vdim"], "rot": {"dims": rt["dim"], "base": 10000.0},
                         "decay": [1.0 - 2.0 ** (-5 - 5.0 * i / max(1, rt["heads"] - 1)) for i in range(rt["heads"])]},
               "left_scale": 1.0, "right_scale": 1.0}},
  ]
  layers = [kinds[i % 3] for i in range(L)]
  fam = {"architecture": "Famupel", "vocab": COMPARE_VOCAB, "width": W, "norm": {"eps": 1e-6}, "streams": size["streams"], "layers": layers,
         "low_ranks": {f"l{i}.decay": gl["rank"] for i in range(L) if i % 3 != 2}}
  return {"vugudra": vugudra_configs(size)["vugudra"], "famupel": fam}


def _famupel_groups(times: dict) -> dict:
  import re
  g = {"attention": 0.0, "dense_products": 0.0, "linear_attention": 0.0, "streams": 0.0, "other": 0.0}
  for name, us in times.items():
    if re.search(r"decode_tma_kernel|decode_cluster_kernel|decode_split_kernel|decode_merge|attention_prefill|attention_generic", name):
      g["attention"] += us
    elif re.search(r"linear_prepare|linear_recurrence|linear_carry|linear_output", name):
      g["linear_attention"] += us
    elif "hyper_connection" in name:
      g["streams"] += us
    elif "gemm_skinny" in name or "gemm_tc_kernel" in name or "gemm_stream_tc" in name or \
        ("anonymous namespace" not in name and re.search(r"nvjet|cutlass|cublas|gemm|gemv|xmma", name, re.I)):
      g["dense_products"] += us
    elif not name.startswith("Memcpy") and not name.startswith("Memset"):
      g["other"] += us
  return g


def famupel_one(name: str, cfg: dict, size: dict, batch: int, steps: int, warmup: int, pk: dict, kernels: bool) -> dict:
  """Prefill and decode of one model of the comparison; with ``kernels`` the device time of its kinds of kernels and the
  rates they reach against the measured peaks (run with dependent launch off, see main)."""
  if name == "vugudra":
    return vugudra_one(name, cfg, size, batch, steps, warmup, pk, kernels)
  import torch
  from miniinfer_b200.engine import StepItem
  from miniinfer_b200.sampling import Sampler, SamplingParams
  W, H, G, hd, L = size["width"], size["heads"], size["kv_heads"], size["head"], size["layers"]
  T = PREFILL_TOKENS
  with tempfile.TemporaryDirectory() as d:
    with open(os.path.join(d, "config.json"), "w") as f:
      json.dump(cfg, f)
    engine = build_engine(d, batch)
    if not kernels:
      dec = time_decode(engine, batch, steps, warmup)
      pre = time_prefill(engine)
      out = {"decode_tok_s": round(dec["tok_s"], 1), "decode_ms": round(dec["ms"], 4), "launches_per_decode_step": int(dec["launches_per_step"]),
             "prefill_tok_s": round(T / (pre["ms"] * 1e-3), 1), "prefill_ms": round(pre["ms"], 3)}
    else:
      rids = fill_context(engine, batch, CONTEXT, seed=1000 + batch)
      params = [SamplingParams(temperature=0.6, max_tokens=GENERATED, ignore_eos=True)] * batch
      tokens_dev = torch.zeros(max(batch, 1), dtype=torch.int32, device="cuda:0")

      def decode(i):
        extras = Sampler.pack(params, list(range(batch)), [i] * batch)
        engine.runner.step_and_sample([StepItem(r, [1], (0,)) for r in rids], extras, Sampler.sample, tokens_dev,
                                      sampling_pad=Sampler.PAD_ROWS)

      for i in range(4):
        decode(i)
      torch.cuda.synchronize()
      dtimes = _kernel_times(lambda i: decode(10 + i), 4)
      dk = _famupel_groups(dtimes)
      for r in rids:
        engine.cache.release_request(r)
      g = torch.Generator().manual_seed(7)

      def whole(i):
        rid = f"rates{i}"
        engine.cache.admit(rid)
        engine.runner.step([StepItem(rid, torch.randint(0, COMPARE_VOCAB, (T,), generator=g).tolist(), (T - 1,))])
        engine.cache.release_request(rid)

      for i in range(2):
        whole(i)
      torch.cuda.synchronize()
      ptimes = _kernel_times(lambda i: whole(10 + i), 2)
      pt = _famupel_groups(ptimes)
      for grp in (pt, dk):
        for key in grp:
          grp[key] = max(grp[key], 1e-9)
      gl, rt, S = size["gla"], size["ret"], size["streams"]
      n_side, n_gla = L // 3, L - L // 3
      ff_w = L * 2 * (size["ff"] * 3 // 2) * W
      seen_all = sum(t + 1 for t in range(T))
      attn_flops = n_side * 4.0 * H * hd * seen_all
      attn_bytes = batch * CONTEXT * n_side * 2 * G * hd * 2
      gh, gd, gv, rk = gl["heads"], gl["dim"], gl["vdim"], gl["rank"]
      rh, rd, rv = rt["heads"], rt["dim"], rt["vdim"]
      gla_w = (rk + 2 * gh * gd + 2 * gh * gv) * W + gh * gd * rk + W * gh * gv
      left_w = (2 * H + 2 * G) * hd * W + W * H * hd
      right_w = (2 * rh * rd + 2 * rh * rv) * W + W * rh * rv
      proj_w = n_gla * gla_w + n_side * (left_w + right_w)
      # what the recurrences must move: queries, keys, values, gates and outputs once (2 bytes a value), the decays' logits
      # (4 bytes) and, in a decode step, every request's state in and out (4 bytes a value)
      lin_io = n_gla * ((2 * gh * gd + 3 * gh * gv) * 2 + gh * gd * 4) + n_side * (2 * rh * rd + 3 * rh * rv) * 2
      lin_state = (n_gla * gh * gd * gv + n_side * rh * rd * rv) * 4 * 2
      # the streams: every sublayer reads and writes S float32 rows of the width, reads the sublayer's output and writes its input
      sublayers = 2 * L
      stream_bytes = sublayers * (2 * S * W * 4 + 2 * W * 2)
      dense_w = ff_w + proj_w + COMPARE_VOCAB * W
      out = {"prefill_attention": {"us": round(pt["attention"], 1), "TFLOP/s": round(attn_flops / pt["attention"] / 1e6, 1),
                                   "frac": round(attn_flops / pt["attention"] / 1e6 / pk["bf16_tflops"], 4)},
             "decode_attention": {"us": round(dk["attention"], 1), "GB/s": round(attn_bytes / dk["attention"] / 1e3, 1),
                                  "frac": round(attn_bytes / dk["attention"] / 1e3 / pk["hbm_gbs"], 4)},
             "prefill_dense_products": {"us": round(pt["dense_products"], 1),
                                        "TFLOP/s": round(2.0 * T * (ff_w + proj_w) / pt["dense_products"] / 1e6, 1),
                                        "frac": round(2.0 * T * (ff_w + proj_w) / pt["dense_products"] / 1e6 / pk["bf16_tflops"], 4)},
             "decode_dense_products": {"us": round(dk["dense_products"], 1), "GB/s": round(2.0 * dense_w / dk["dense_products"] / 1e3, 1),
                                       "frac": round(2.0 * dense_w / dk["dense_products"] / 1e3 / pk["hbm_gbs"], 4)},
             "prefill_linear_attention": {"us": round(pt["linear_attention"], 1), "GB/s": round(T * lin_io / pt["linear_attention"] / 1e3, 1),
                                          "frac": round(T * lin_io / pt["linear_attention"] / 1e3 / pk["hbm_gbs"], 4)},
             "decode_linear_attention": {"us": round(dk["linear_attention"], 1),
                                         "GB/s": round(batch * (lin_io + lin_state) / dk["linear_attention"] / 1e3, 1),
                                         "frac": round(batch * (lin_io + lin_state) / dk["linear_attention"] / 1e3 / pk["hbm_gbs"], 4)},
             "prefill_streams": {"us": round(pt["streams"], 1), "GB/s": round(T * stream_bytes / pt["streams"] / 1e3, 1),
                                 "frac": round(T * stream_bytes / pt["streams"] / 1e3 / pk["hbm_gbs"], 4)},
             "decode_streams_us": round(dk["streams"], 1),
             "other_us": {"prefill": round(pt["other"], 1), "decode": round(dk["other"], 1)}}

      def top(times):
        rows = sorted(((us, n) for n, us in times.items() if not n.startswith("Mem")), reverse=True)[:14]
        return [[round(us, 1), n.replace("(anonymous namespace)::", "")[:70]] for us, n in rows]

      out["top_kernels_us"] = {"prefill": top(ptimes), "decode": top(dtimes)}
    engine.stop()
    del engine
    gc.collect()
    torch.cuda.empty_cache()
  return out


# ---------------------------------------------------------------------------------------------- --compare luporax
# Sizes for the comparison of the Luporax design with the closest design the engine has, Rikanex (attention with shaped
# weights and routed experts in every layer but the first), at equal size: the sizes of the Rikanex comparison - width,
# heads, experts (count, width, per token), layers, vocabulary.  Luporax's layers go attention, real-gated linear recurrent
# unit, minimal gated recurrence, and again; every layer has the routed experts and a shared expert of an expert's width;
# its attention sees every earlier token (the design has no window), Rikanex's the last 1024.
LUPORAX_RGLRU_BLOCKS = 8


def luporax_configs(size: dict) -> dict:
  W, H, G, hd, L = size["width"], size["heads"], size["kv_heads"], size["head"], size["layers"]
  mlp = {"kind": "moe", "expert": {"ff": size["expert_ff"], "limit": 7.0}, "router": {"experts": size["experts"], "top": size["top"]},
         "shared": {"ff": size["expert_ff"], "limit": 7.0}}
  kinds = [
    {"type": "attention", "mlp": mlp, "mixer": {"heads": H, "kv_heads": G, "dim": hd, "vdim": hd, "scale": hd ** -0.5, "softcap": 50.0,
                                                "rot": {"dims": hd, "base": 500000.0}}},
    {"type": "rglru", "mlp": mlp, "mixer": {"width": W, "blocks": LUPORAX_RGLRU_BLOCKS, "conv": 4}},
    {"type": "mingru", "mlp": mlp, "mixer": {"width": W}},
  ]
  lup = {"architecture": "Luporax", "vocab": COMPARE_VOCAB, "width": W, "norm": {"eps": 1e-6}, "residual_mult": 0.7, "logit_scale": 0.25,
         "layers": [kinds[i % 3] for i in range(L)]}
  return {"rikanex": compare_configs(size)["rikanex"], "luporax": lup}


def _luporax_groups(times: dict) -> dict:
  import re
  g = {"attention": 0.0, "experts": 0.0, "routing": 0.0, "dense_products": 0.0, "recurrence": 0.0, "block": 0.0, "other": 0.0}
  for name, us in times.items():
    if re.search(r"decode_tma_kernel|decode_cluster_kernel|decode_split_kernel|decode_merge|attention_prefill|attention_generic", name):
      g["attention"] += us
    elif "moe_gemm" in name or "moe_stream" in name or re.search(r"gemm_tc_kernel<\w+, \w+, (true|\(bool\)1)[,>]", name):
      g["experts"] += us
    elif re.search(r"moe_route|moe_align|moe_combine|moe_gather", name):
      g["routing"] += us
    elif re.search(r"diag_recurrence|causal_conv|conv_state|gemm_batched", name):
      g["recurrence"] += us
    elif re.search(r"token_shift|norm_scaled_add", name):
      g["block"] += us
    elif "gemm_skinny" in name or "gemm_tc_kernel" in name or "gemm_stream_tc" in name or \
        ("anonymous namespace" not in name and re.search(r"nvjet|cutlass|cublas|gemm|gemv|xmma", name, re.I)):
      g["dense_products"] += us
    elif not name.startswith("Memcpy") and not name.startswith("Memset"):
      g["other"] += us
  return g


def luporax_one(name: str, cfg: dict, size: dict, batch: int, steps: int, warmup: int, pk: dict, kernels: bool) -> dict:
  """Prefill and decode of one model of the comparison; with ``kernels`` the device time of its kinds of kernels and the
  rates they reach against the measured peaks (run with dependent launch off, see main)."""
  if name == "rikanex":
    return compare_one(name, cfg, size, batch, steps, warmup, pk, kernels)
  import torch
  from miniinfer_b200.engine import StepItem
  from miniinfer_b200.sampling import Sampler, SamplingParams
  W, H, G, hd, L = size["width"], size["heads"], size["kv_heads"], size["head"], size["layers"]
  T = PREFILL_TOKENS
  with tempfile.TemporaryDirectory() as d:
    with open(os.path.join(d, "config.json"), "w") as f:
      json.dump(cfg, f)
    engine = build_engine(d, batch)
    if not kernels:
      dec = time_decode(engine, batch, steps, warmup)
      pre = time_prefill(engine)
      out = {"decode_tok_s": round(dec["tok_s"], 1), "decode_ms": round(dec["ms"], 4), "launches_per_decode_step": int(dec["launches_per_step"]),
             "prefill_tok_s": round(T / (pre["ms"] * 1e-3), 1), "prefill_ms": round(pre["ms"], 3)}
    else:
      rids = fill_context(engine, batch, CONTEXT, seed=1000 + batch)
      params = [SamplingParams(temperature=0.6, max_tokens=GENERATED, ignore_eos=True)] * batch
      tokens_dev = torch.zeros(max(batch, 1), dtype=torch.int32, device="cuda:0")

      def decode(i):
        extras = Sampler.pack(params, list(range(batch)), [i] * batch)
        engine.runner.step_and_sample([StepItem(r, [1], (0,)) for r in rids], extras, Sampler.sample, tokens_dev,
                                      sampling_pad=Sampler.PAD_ROWS)

      for i in range(4):
        decode(i)
      torch.cuda.synchronize()
      dtimes = _kernel_times(lambda i: decode(10 + i), 4)
      dk = _luporax_groups(dtimes)
      touched = float(size["experts"])
      for gph in engine.runner._graphs.values():      # what the last step's last routed layer did read: the row tiles that an expert owns
        buf = gph.ws._bufs.get(("moe_tile_expert", torch.int32))
        if buf is not None:
          touched = float((buf >= 0).sum().item())
      for r in rids:
        engine.cache.release_request(r)
      g = torch.Generator().manual_seed(7)

      def whole(i):
        rid = f"rates{i}"
        engine.cache.admit(rid)
        engine.runner.step([StepItem(rid, torch.randint(0, COMPARE_VOCAB, (T,), generator=g).tolist(), (T - 1,))])
        engine.cache.release_request(rid)

      for i in range(2):
        whole(i)
      torch.cuda.synchronize()
      ptimes = _kernel_times(lambda i: whole(10 + i), 2)
      pt = _luporax_groups(ptimes)
      for grp in (pt, dk):
        for key in grp:
          grp[key] = max(grp[key], 1e-9)
      n_att, n_rg, n_mg = (L + 2) // 3, (L + 1) // 3, L // 3
      E, F, top = size["experts"], size["expert_ff"], size["top"]
      attn_flops = n_att * 4.0 * H * hd * sum(t + 1 for t in range(T))
      attn_bytes = batch * CONTEXT * n_att * 2 * G * hd * 2
      moe_flops = L * T * top * 3 * 2.0 * F * W
      moe_bytes = L * touched * 3 * F * W * 2
      proj_w = n_att * ((H + 2 * G) * hd * W + W * H * hd) + n_rg * 3 * W * W + n_mg * 4 * W * W
      shared_w = L * 3 * F * W
      dense_w = proj_w + shared_w + COMPARE_VOCAB * W
      # what the recurrent layers must move a token besides their dense products: the convolution (x in, u out), the gates'
      # batched product (u in, two float32 logits a channel out) and the recurrence (u, logits, y in, the read-out out) of an
      # rglru layer - 28 bytes a channel -, z, x, g in and the read-out out of a mingru layer - 8 bytes a channel; in a decode
      # step also every request's states in and out (4 bytes a value; the convolution keeps three earlier inputs a channel)
      rec_io = n_rg * 28 * W + n_mg * 8 * W
      rec_state = (n_rg * 4 * W + n_mg * W) * 4 * 2
      gates_flops = n_rg * T * 2.0 * 2 * W * (W // LUPORAX_RGLRU_BLOCKS)
      # the blocks: a sublayer reads the float32 row and writes its rounding (the mixer's through the shift), then reads the
      # sublayer's output and the row and writes the row (and its rounding for the next sublayer)
      block_bytes = L * ((4 + 2) * W + (2 + 4 + 4 + 2) * W + (2 + 4 + 4) * W)
      out = {"prefill_attention": {"us": round(pt["attention"], 1), "TFLOP/s": round(attn_flops / pt["attention"] / 1e6, 1),
                                   "frac": round(attn_flops / pt["attention"] / 1e6 / pk["bf16_tflops"], 4)},
             "decode_attention": {"us": round(dk["attention"], 1), "GB/s": round(attn_bytes / dk["attention"] / 1e3, 1),
                                  "frac": round(attn_bytes / dk["attention"] / 1e3 / pk["hbm_gbs"], 4)},
             "prefill_experts": {"us": round(pt["experts"], 1), "TFLOP/s": round(moe_flops / pt["experts"] / 1e6, 1),
                                 "frac": round(moe_flops / pt["experts"] / 1e6 / pk["bf16_tflops"], 4)},
             "decode_experts": {"us": round(dk["experts"], 1), "GB/s": round(moe_bytes / dk["experts"] / 1e3, 1),
                                "frac": round(moe_bytes / dk["experts"] / 1e3 / pk["hbm_gbs"], 4), "experts_read_per_layer": round(touched, 1)},
             "routing_us": {"prefill": round(pt["routing"], 1), "decode": round(dk["routing"], 1)},
             "prefill_dense_products": {"us": round(pt["dense_products"], 1),
                                        "TFLOP/s": round(2.0 * T * (proj_w + shared_w) / pt["dense_products"] / 1e6, 1),
                                        "frac": round(2.0 * T * (proj_w + shared_w) / pt["dense_products"] / 1e6 / pk["bf16_tflops"], 4)},
             "decode_dense_products": {"us": round(dk["dense_products"], 1), "GB/s": round(2.0 * dense_w / dk["dense_products"] / 1e3, 1),
                                       "frac": round(2.0 * dense_w / dk["dense_products"] / 1e3 / pk["hbm_gbs"], 4)},
             "prefill_recurrence": {"us": round(pt["recurrence"], 1), "GB/s": round(T * rec_io / pt["recurrence"] / 1e3, 1),
                                    "frac": round(T * rec_io / pt["recurrence"] / 1e3 / pk["hbm_gbs"], 4),
                                    "gates_GFLOP": round(gates_flops / 1e9, 2)},
             "decode_recurrence": {"us": round(dk["recurrence"], 1), "GB/s": round(batch * (rec_io + rec_state) / dk["recurrence"] / 1e3, 1),
                                   "frac": round(batch * (rec_io + rec_state) / dk["recurrence"] / 1e3 / pk["hbm_gbs"], 4)},
             "prefill_block": {"us": round(pt["block"], 1), "GB/s": round(T * block_bytes / pt["block"] / 1e3, 1),
                               "frac": round(T * block_bytes / pt["block"] / 1e3 / pk["hbm_gbs"], 4)},
             "decode_block_us": round(dk["block"], 1),
             "other_us": {"prefill": round(pt["other"], 1), "decode": round(dk["other"], 1)}}

      def top_of(times):
        rows = sorted(((us, n) for n, us in times.items() if not n.startswith("Mem")), reverse=True)[:14]
        return [[round(us, 1), n.replace("(anonymous namespace)::", "")[:70]] for us, n in rows]

      out["top_kernels_us"] = {"prefill": top_of(ptimes), "decode": top_of(dtimes)}
    engine.stop()
    del engine
    gc.collect()
    torch.cuda.empty_cache()
  return out


def compare_designs(args) -> int:
  """``--compare rikanex`` / ``--compare vugudra``: the design beside the Qwen3 dense decoder at equal sizes (random weights);
  ``--compare famupel``: the design beside Vugudra, ``--compare luporax``: the design beside Rikanex, each the closest of
  the engine's designs, at equal sizes: prefill of
  one 2048-token prompt and decode steps at ``--batch`` requests with ``--context``-token contexts, and, from a process of
  its own with dependent launch off, what the kinds of kernels of both reach against the measured peaks."""
  pk = peaks()
  warmup = max(args.warmup, 3)
  global GENERATED, MAX_MODEL_LEN
  GENERATED = max(GENERATED, warmup + args.steps + args.batch * -(-CONTEXT // PREFILL_TOKENS) + 64)
  MAX_MODEL_LEN = max(MAX_MODEL_LEN, -(-(CONTEXT + GENERATED + 128) // 1024) * 1024)
  sizes = [x for x in args.sizes.split(",") if x]
  design = args.compare
  sizes_of, configs_of, one = {"rikanex": (COMPARE_SIZES, compare_configs, compare_one), "vugudra": (VUGUDRA_SIZES, vugudra_configs, vugudra_one),
                               "famupel": (FAMUPEL_SIZES, famupel_configs, famupel_one),
                               "luporax": (COMPARE_SIZES, luporax_configs, luporax_one)}[design]
  beside = {"famupel": "vugudra", "luporax": "rikanex"}.get(design, "qwen3")
  result = {"compare": f"{design} beside {beside} at equal sizes", "batch": args.batch, "context": CONTEXT, "window": COMPARE_WINDOW,
            "vocab": COMPARE_VOCAB, "prefill_tokens": PREFILL_TOKENS, "steps": args.steps, "warmup": warmup, "dtype": "bf16",
            "data": "synthetic: random weights, uniform random token ids", "peaks": pk["source"], "sizes": {}}
  kernels_child = args.impl == "compare-child"
  clocks = None if kernels_child else ClockSampler()
  if clocks:
    clocks.start()
  for tag in sizes:
    size = sizes_of[tag]
    row = {"size": size}
    for name, cfg in configs_of(size).items():
      row[name] = one(name, cfg, size, args.batch, args.steps, warmup, pk, kernels_child)
    result["sizes"][tag] = row
  if clocks:
    result["clocks"] = clocks.stop()
  if not kernels_child and not args.skip_kernels:
    cmd = [sys.executable, os.path.abspath(__file__), "--impl", "compare-child", "--compare", design, "--sizes", args.sizes,
           "--batch", str(args.batch), "--context", str(CONTEXT), "--steps", str(args.steps), "--warmup", str(warmup)]
    proc = subprocess.run(cmd, capture_output=True, text=True, env=dict(os.environ, MINIINFER_B200_PDL="0"))
    found = [l for l in proc.stdout.splitlines() if l.startswith('{"compare"')]
    if found:
      child = json.loads(found[-1])
      for tag in sizes:
        for name in (beside, design):
          result["sizes"][tag][name]["kernels"] = child["sizes"][tag][name]
    else:
      result["kernels_unavailable"] = (proc.stderr or "no output").strip().splitlines()[-1][:300]
  print(json.dumps(result))
  return 0


def main() -> int:
  global CONTEXT
  ap = argparse.ArgumentParser()
  ap.add_argument("--gpus", type=int, default=1)
  ap.add_argument("--steps", type=int, default=128)
  ap.add_argument("--warmup", type=int, default=8)
  ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-child", "kernels-child", "compare-child"])
  ap.add_argument("--compare", default=None, choices=["rikanex", "vugudra", "famupel", "luporax"],
                  help="time the Rikanex or the Vugudra design beside the Qwen3 dense decoder, the Famupel design beside Vugudra, or the Luporax design beside Rikanex, at equal sizes (--sizes), print one JSON line and exit")
  ap.add_argument("--sizes", default="s,m,l", help="with --compare: which of the sizes s, m, l (commas between them)")
  ap.add_argument("--batch", type=int, default=8)
  ap.add_argument("--shape", default="0.6b", choices=sorted(SHAPES), help="layer sizes: the default, or another Qwen3 model's")
  ap.add_argument("--layers", type=int, default=None, help="fewer layers than the model has (named in config)")
  ap.add_argument("--context", type=int, default=None, help="tokens each request holds when decoding starts (default 2048; 32b: 4096)")
  ap.add_argument("--skip-kernels", action="store_true", help="leave out the per-kernel rates")
  ap.add_argument("--skip-points", action="store_true")
  ap.add_argument("--mixed", action="store_true",
                  help="run a continuous batch of 64 requests through LLMEngine.generate, print its throughput and exit")
  ap.add_argument("--kernel-case", default=None, choices=KERNEL_CASES,
                  help="run one kernel alone on an input larger than L2 (the workload of the ncu summaries) and exit")
  ap.add_argument("--kernel-table", nargs="?", const="decode", default=None, choices=["decode", "prefill"],
                  help="print the device time of each kernel of a decode step (default) or a prefill step and exit")
  args = ap.parse_args()
  if args.kernel_case:
    print(kernel_case(args.kernel_case))
    return 0
  if args.compare:
    if args.context is not None:
      CONTEXT = args.context
    return compare_designs(args)
  if args.impl == "reference":
    return reference_arm(args)
  if args.impl == "reference-child":
    return reference_child(args)
  MODEL.update(SHAPES[args.shape])
  shape_name = f"Qwen3-{args.shape.upper()} shape"
  if args.layers is None:
    args.layers = MODEL["num_hidden_layers"]
  if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
    print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
    return 2

  import torch
  pk = peaks()
  cfg = dict(MODEL, num_hidden_layers=args.layers)
  warmup = max(args.warmup, 3)
  # room for the tokens that the timed steps generate, whatever --steps says
  global GENERATED, MAX_MODEL_LEN
  CONTEXT = args.context if args.context is not None else SHAPE_CONTEXT.get(args.shape, CONTEXT)
  MAX_MODEL_LEN = max(MAX_MODEL_LEN, SHAPE_MAX_MODEL_LEN.get(args.shape, 0))
  GENERATED = max(GENERATED, warmup + args.steps + args.batch * -(-CONTEXT // PREFILL_TOKENS) + 64)
  MAX_MODEL_LEN = max(MAX_MODEL_LEN, -(-(CONTEXT + GENERATED + 128) // 1024) * 1024)
  cfg["max_position_embeddings"] = max(cfg.get("max_position_embeddings", 0), MAX_MODEL_LEN)
  with tempfile.TemporaryDirectory() as d:
    with open(os.path.join(d, "config.json"), "w") as f:
      json.dump(cfg, f)
    if args.mixed:
      print(json.dumps(dict(mixed_workload(d), layers=args.layers, model=shape_name)))
      return 0
    if args.kernel_table:
      print(kernel_table(build_engine(d, args.batch), args.batch, mode=args.kernel_table))
      return 0
    if args.impl == "kernels-child":
      print(json.dumps({"kernels": kernel_rates(build_engine(d, args.batch), args.batch, cfg, args.layers, pk)}))
      return 0
    clocks = ClockSampler()
    engine = build_engine(d, args.batch)
    clocks.start()
    dec = time_decode(engine, args.batch, args.steps, warmup)
    e2e = time_e2e(engine, args.batch, args.steps, warmup)
    pre = time_prefill(engine)
    clock_info = clocks.stop()
    points = {}
    if not args.skip_points:
      for b in (1, 64):
        engine.stop()
        del engine
        gc.collect()
        torch.cuda.empty_cache()
        engine = build_engine(d, b)
        points[f"decode_b{b}"] = round(time_decode(engine, b, args.steps, warmup)["tok_s"], 1)

    # Per-kernel times come from a process of its own with dependent launch off: with it on, a kernel is placed
    # while its predecessor runs and the time it spends waiting there would count as its own.
    rates = None
    if not args.skip_kernels:
      engine.stop()
      del engine
      gc.collect()
      torch.cuda.empty_cache()
      cmd = [sys.executable, os.path.abspath(__file__), "--impl", "kernels-child", "--shape", args.shape, "--batch", str(args.batch),
             "--layers", str(args.layers), "--context", str(CONTEXT)]
      proc = subprocess.run(cmd, capture_output=True, text=True, env=dict(os.environ, MINIINFER_B200_PDL="0"))
      found = [l for l in proc.stdout.splitlines() if l.startswith('{"kernels"')]
      rates = json.loads(found[-1])["kernels"] if found else {"unavailable": (proc.stderr or "no output").strip().splitlines()[-1][:200]}

  mb = model_bytes(cfg, args.layers)
  step_bytes = mb["weights"] + args.batch * dec["mean_ctx"] * mb["kv_per_token"]
  achieved = step_bytes / (dec["ms"] * 1e-3) / 1e9
  flops = prefill_flops(cfg, args.layers, PREFILL_TOKENS)
  line = {
    "metric": f"decode tok/s at batch {args.batch} (Qwen3-{args.shape.upper()} shape, {CONTEXT}-token contexts)",
    "value": round(dec["tok_s"], 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
    "ms_per_step": round(dec["ms"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
    "dtype": "bf16", "data": "synthetic: random weights N(0, 0.02), uniform random token ids", "impl": "ours",
    "config": {"model": shape_name, "layers": args.layers, "layers_of_model": MODEL["num_hidden_layers"],
               "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
               "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
               "tied_head": bool(cfg["tie_word_embeddings"]), "global_batch": args.batch, "seq_len": CONTEXT, "generated": GENERATED,
               "max_model_len": MAX_MODEL_LEN, "page_size": PAGE, "parallelism": "single GPU",
               "l2": "each step reads weights+cache (>1 GB), larger than L2", "sampling": "temperature 0.6",
               "decode_path": "CUDA graph replay; e2e: a step is launched before the tokens of the step before are read (enable_overlap)"},
    "e2e": {"value": round(e2e["tok_s"], 1), "unit": "tok/s", "ms_per_step": round(e2e["ms"], 4),
            "h2d_bytes_per_step": int(e2e["h2d"]), "d2h_bytes_per_step": int(e2e["d2h"])},
    "gpu_launches": int(dec["launches_per_step"] * args.steps),
    "launches_per_step": int(dec["launches_per_step"]),
    "prefill": {"value": round(PREFILL_TOKENS / (pre["ms"] * 1e-3), 1), "tokens": PREFILL_TOKENS, "ms": round(pre["ms"], 3),
                "frac": round(flops / (pre["ms"] * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
    "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                 "frac": round(achieved / pk["hbm_gbs"], 4), "peaks": pk["source"]},
    "points": points,
    "kernels": rates,
    "clocks": clock_info,
  }
  print(json.dumps(line))
  return 0


if __name__ == "__main__":
  sys.exit(main())
