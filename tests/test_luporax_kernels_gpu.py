"""Each mechanism of the Luporax design alone: the engine's operation, run over a step cut in several ways, against the
plain function of tests/plain_luporax.py on the whole sequence.  Inputs are made so that a fault shows: one key far back
whose score stands out, decays near 0 and near 1, states of other requests that must be left alone, sizes that are no
powers of two and values that a model may happen to make equal or 1."""
import math
from types import SimpleNamespace

import pytest
import torch

import plain_luporax as plain
from gpu_helpers import DEV, make_attention_case

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def tol(dtype):
  return 3e-5 if dtype == "float32" else 3e-2


def step_ctx(items):
  """The description of a step: ``items`` = (new tokens, position of the first of them, state slot) for each request."""
  q_len = [n for n, _, _ in items]
  q_start = [sum(q_len[:i]) for i in range(len(q_len))]
  dev = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
  return SimpleNamespace(q_start=dev(q_start), q_len=dev(q_len), seq_slot=dev([s for _, _, s in items]), num_items=len(items),
                         num_tokens=sum(q_len), token_item=dev([b for b, n in enumerate(q_len) for _ in range(n)]),
                         positions=dev([p0 + i for n, p0, _ in items for i in range(n)]))


def cuts_of(T, sizes):
  out, pos, k = [], 0, 0
  while pos < T:
    n = min(sizes[k % len(sizes)], T - pos)
    out.append(n)
    pos += n
    k += 1
  return out


def rounded(t, dtype):
  return t.to(DT[dtype]).float()


def in_portions(T, cuts, run, width, dtype, state, slot=2):
  """Runs ``run(rows, ctx) -> out rows`` over one request's tokens in portions; beside it in every step a one-token item of
  another request in slot 0.  Slot 1 is nobody's and must be left alone."""
  state[1].fill_(7.0)
  got = torch.zeros((T, width), dtype=DT[dtype], device=DEV)
  pos = 0
  for n in cuts:
    rows = torch.cat((torch.arange(pos, pos + n), torch.tensor([0])))
    out = run(rows, step_ctx([(n, pos, slot), (1, 0, 0)]))
    got[pos:pos + n] = out[:n]
    pos += n
  assert pos == T and float((state[1] - 7.0).abs().max()) == 0
  return got.float().cpu()


CUTS = [None, (1,), (2,), (13, 7, 2, 29, 3, 2, 5, 17, 2, 64, 1, 2)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("C", [8, 40, 96, 200])
def test_mingru_recurrence_against_the_plain_one(dtype, C):
  from miniinfer_b200.kernels import ops
  g = torch.Generator().manual_seed(C)
  T = 150
  proj = torch.randn((T, 3 * C), generator=g) * 2.0
  proj[:, :C // 2] -= 6.0                                  # gates near 0: a memory of hundreds of tokens
  proj[:, C // 2:C // 2 + 2] += 12.0                       # gates near 1: nothing is kept
  proj = rounded(proj, dtype)
  zb, xb = torch.randn(C, generator=g) * 0.5, torch.randn(C, generator=g) * 0.5
  z = torch.sigmoid(proj[:, :C].double() + zb.double())
  x = proj[:, C:2 * C].double() + xb.double()
  S = plain.diagonal_recurrence(1.0 - z, z * torch.where(x >= 0, x + 0.5, torch.sigmoid(x)))
  want = (S * plain.silu(proj[:, 2 * C:].double())).float()
  for sizes in CUTS:
    state = torch.zeros((4, C + 5), dtype=torch.float32, device=DEV)

    def run(rows, ctx):
      out = torch.zeros((len(rows), C), dtype=DT[dtype], device=DEV)
      ops.mingru_recurrence(out, proj[rows].to(DT[dtype]).to(DEV), zb.to(DEV), xb.to(DEV), state, ctx)
      return out

    got = in_portions(T, cuts_of(T, sizes) if sizes else [T], run, C, dtype, state)
    assert float((got - want).abs().max()) <= tol(dtype) * float(want.abs().max()), f"cuts {sizes}"
    assert float((state[2, :C].cpu() - S[-1].float()).abs().max()) <= 3e-5 * float(S.abs().max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("C,blocks", [(8, 1), (40, 5), (96, 2), (192, 3)])
def test_rglru_recurrence_against_the_plain_one(dtype, C, blocks):
  from miniinfer_b200.kernels import ops
  g = torch.Generator().manual_seed(C + blocks)
  T, P = 150, C // blocks
  u = rounded(torch.randn((T, C), generator=g), dtype)
  y = rounded(torch.randn((T, C), generator=g), dtype)
  gates = torch.randn((T, blocks, 2 * P), generator=g) * 2.0          # float32 logits, a part's r then its i
  rb, ib, yb = (torch.randn(C, generator=g) * 0.5 for _ in range(3))
  lam = -3.5 + 2.0 * torch.randn(C, generator=g)
  lam[0], lam[-1] = -12.0, 4.0                                        # a decay of 1 to six digits, and one that forgets at once
  r = torch.sigmoid(gates[:, :, :P].reshape(T, C).double() + rb.double())
  i = torch.sigmoid(gates[:, :, P:].reshape(T, C).double() + ib.double())
  a = torch.exp(-8.0 * r * torch.nn.functional.softplus(lam.double()))
  S = plain.diagonal_recurrence(a, torch.sqrt(1.0 - a * a) * i * u.double())
  want = (S * plain.gelu_tanh(y.double() + yb.double())).float()
  for sizes in CUTS:
    state = torch.zeros((4, C), dtype=torch.float32, device=DEV)

    def run(rows, ctx):
      out = torch.zeros((len(rows), C), dtype=DT[dtype], device=DEV)
      ops.rglru_recurrence(out, u[rows].to(DT[dtype]).to(DEV), gates[rows].reshape(len(rows), 2 * C).contiguous().to(DEV),
                           y[rows].to(DT[dtype]).to(DEV), rb.to(DEV), ib.to(DEV), yb.to(DEV), lam.to(DEV), state, ctx, blocks)
      return out

    got = in_portions(T, cuts_of(T, sizes) if sizes else [T], run, C, dtype, state)
    assert float((got - want).abs().max()) <= tol(dtype) * float(want.abs().max()), f"cuts {sizes}"
    assert float((state[2].cpu() - S[-1].float()).abs().max()) <= 3e-5 * float(S.abs().max())


@pytest.mark.skipif(DEV == "cpu", reason="two forms of the CUDA kernel")
@pytest.mark.parametrize("C", [40, 256])
def test_long_portions_in_stretches_side_by_side_agree_with_the_walk_in_order(C, monkeypatch):
  """A bfloat16 step of long portions takes the form with stretches side by side; its outputs and end states are those of
  the walk in order (up to float32 rounding of the chained maps), also for a request that starts from a state, beside a
  short request that the segmented launch walks in order."""
  from miniinfer_b200.kernels import ops
  g = torch.Generator().manual_seed(3)
  T = 2 * 800 + 3
  proj = (torch.randn((T, 3 * C), generator=g) * 2.0).to(torch.bfloat16).to(DEV)
  proj[:, :C // 2] -= 5.0
  zb, xb = (torch.randn(C, generator=g) * 0.5).to(DEV), (torch.randn(C, generator=g) * 0.5).to(DEV)
  from miniinfer_b200.engine.context import Workspace
  outs, states = [], []
  for segments, ws in (("1", Workspace(torch.device(DEV))), ("0", None), ("1", None)):      # prepared and walked, in order, walked as it is made
    monkeypatch.setenv("MINIINFER_B200_RECURRENCE_SEGMENTS", segments)
    state = torch.zeros((4, C), dtype=torch.float32, device=DEV)
    state[3] = torch.linspace(-1, 1, C)
    out = torch.zeros((T, C), dtype=torch.bfloat16, device=DEV)
    ctx = step_ctx([(800, 0, 2), (3, 0, 0), (800, 50, 3)])
    assert ops._recurrence_segmented(torch.bfloat16, ctx) == int(segments)
    ops.mingru_recurrence(out, proj, zb, xb, state, ctx, workspace=ws)
    outs.append(out.float().cpu())
    states.append(state.cpu())
  for k in (0, 2):
    assert float((outs[k] - outs[1]).abs().max()) <= 2e-2 * float(outs[1].abs().max())
    assert float((states[k] - states[1]).abs().max()) <= 1e-4 * float(states[1].abs().max())
  assert torch.equal(outs[2][800:803], outs[1][800:803])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("W", [24, 64, 257 * 4])
def test_token_shift_and_the_norm_of_a_sublayers_output(dtype, W):
  """h = x + (x_before - x) * shift across cuts, the row before a portion coming from the state; then x += mult * norm(y),
  which also leaves the last row - as it was before the addition - as the next portion's predecessor."""
  from miniinfer_b200.kernels import ops
  g = torch.Generator().manual_seed(W)
  T = 70
  x = torch.randn((T, W), generator=g)
  y = rounded(torch.randn((T, W), generator=g) * 3.0, dtype)
  shift, w = torch.rand(W, generator=g), 1.0 + 0.3 * torch.randn(W, generator=g)
  want_h = plain.token_shift(x.double(), shift.double()).float()
  want_x = (x.double() + 0.7 * plain.rms_unit(y.double(), 1e-5) * w.double()).float()
  for sizes in CUTS:
    state = torch.zeros((4, W + 3), dtype=torch.float32, device=DEV)
    resid = x.clone().to(DEV)
    copies = torch.zeros((T, W), dtype=DT[dtype], device=DEV)
    pos = 0
    hs = torch.zeros((T, W), dtype=DT[dtype], device=DEV)
    for n in cuts_of(T, sizes) if sizes else [T]:
      ctx = step_ctx([(n, pos, 2)])
      ops.token_shift(hs[pos:pos + n], resid[pos:pos + n], shift.to(DEV), state, ctx)
      ops.norm_scaled_add(resid[pos:pos + n], y[pos:pos + n].to(DT[dtype]).to(DEV), w.to(DEV), 1e-5, 0.7, ctx,
                          copy=copies[pos:pos + n], keep=state)
      pos += n
    assert float((hs.float().cpu() - want_h).abs().max()) <= (1e-6 if dtype == "float32" else 2e-2) * float(want_h.abs().max())
    assert float((resid.cpu() - want_x).abs().max()) <= 1e-5 * float(want_x.abs().max())
    assert float((copies.float().cpu() - want_x).abs().max()) <= (1e-5 if dtype == "float32" else 1e-2) * float(want_x.abs().max())
    assert torch.equal(state[2, :W].cpu(), x[-1]) and float(state[1].abs().max()) == 0
  plainly = torch.zeros((T, W), dtype=DT[dtype], device=DEV)
  ops.token_shift(plainly, x.to(DEV), None, None, step_ctx([(T, 0, 0)]))
  assert torch.equal(plainly.cpu(), x.to(DT[dtype]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("C,taps", [(8, 1), (40, 3), (96, 4)])
def test_convolution_over_biased_inputs(dtype, C, taps):
  """The inputs of the convolution are the projection plus its bias; before a request's start stand zeros, not the bias."""
  from miniinfer_b200.kernels import ops
  g = torch.Generator().manual_seed(taps)
  T = 60
  x = rounded(torch.randn((T, C), generator=g), dtype)
  w, cb, ib = torch.randn((C, taps), generator=g) * 0.5, torch.randn(C, generator=g), 2.0 + torch.randn(C, generator=g)
  want = plain.causal_conv(x.double() + ib.double(), w.double(), cb.double()).float()
  for sizes in CUTS:
    state = torch.zeros((4, max(1, (taps - 1) * C)), dtype=torch.float32, device=DEV)

    def run(rows, ctx):
      out = torch.zeros((len(rows), C), dtype=DT[dtype], device=DEV)
      ops.causal_conv(out, x[rows].to(DT[dtype]).to(DEV), w.to(DEV), cb.to(DEV), state, ctx, silu=False, in_bias=ib.to(DEV))
      return out

    if taps == 1:
      state = torch.zeros((4, 1), dtype=torch.float32, device=DEV)
      got = torch.zeros((T, C), dtype=DT[dtype], device=DEV)
      got = run(torch.arange(T), step_ctx([(T, 0, 2)])).float().cpu()
    else:
      got = in_portions(T, cuts_of(T, sizes) if sizes else [T], run, C, dtype, state)
    assert float((got - want).abs().max()) <= (1e-5 if dtype == "float32" else 2e-2) * float(want.abs().max()), f"cuts {sizes}"


def plain_sigmoid_attention(qkv, kv, bt, batch, nh, nkv, hd, scale, softcap, bias, sigmoid=True):
  """Every row of the step from the cache, in float64: weights sigmoid(cap(scale q.k) + bias) over the keys 0 .. position."""
  T, P, G = qkv.shape[0], kv.shape[3], nh // nkv
  q = qkv.double().view(T, -1, hd)[:, :nh]
  pos, item, slots = batch.positions.tolist(), batch.token_item.tolist(), batch.seq_slot.tolist()
  out = torch.zeros((T, nh, hd), dtype=torch.float64)
  for t in range(T):
    js = torch.arange(0, pos[t] + 1)
    pages = bt[slots[item[t]]].long()[js // P]
    k = kv[pages, 0, :, js % P, :].double().repeat_interleave(G, dim=1)
    v = kv[pages, 1, :, js % P, :].double().repeat_interleave(G, dim=1)
    s = torch.einsum("hd,nhd->hn", q[t], k) * scale
    if softcap:
      s = softcap * torch.tanh(s / softcap)
    w = torch.sigmoid(s + bias.double()[:, None]) if sigmoid else torch.softmax(s, -1)
    out[t] = torch.einsum("hn,nhd->hd", w, v)
  return out.reshape(T, nh * hd).float()


ATTENTION_CASES = [
  # (context, new tokens) of every request; heads, kv heads, head size, page size
  ([(300, 300), (77, 1), (1, 1), (129, 2)], 4, 2, 64, 64),       # heads of 64 on pages of 64: the tcgen05 prefill and the TMA decode kernel
  ([(200, 1), (64, 1), (65, 1), (1000, 1)], 8, 2, 64, 64),
  ([(130, 67), (40, 1), (16, 16), (17, 1)], 6, 1, 48, 16),       # heads of 48 on pages of 16: the mma.sync prefill and the cp.async decode kernel
  ([(90, 1), (33, 33)], 3, 3, 24, 8),                            # heads of 24: the generic kernel in both dtypes
  ([(300, 300), (77, 1), (700, 1), (129, 2)], 8, 1, 128, 64),    # heads of 128, eight query heads on the one key/value head
  ([(130, 67), (40, 1), (300, 1)], 2, 1, 256, 64),               # heads of 256: beyond the tcgen05 kernel's sizes
  ([(200, 200), (90, 1)], 4, 4, 32, 64),                         # heads of 32 on pages of 64: no tensor copies of half a row
  ([(150, 150), (65, 1), (64, 1)], 10, 5, 80, 16),               # heads of 80
  ([(520, 1), (64, 1)], 32, 2, 64, 64),                          # sixteen query heads on a key/value head: two passes over the tiles
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", range(len(ATTENTION_CASES)))
@pytest.mark.parametrize("softcap", [0.0, 6.0])
def test_sigmoid_weights_and_capped_scores_in_every_attention_kernel(dtype, case, softcap):
  """Weights that are sigmoids of the score plus a number per head, not normalised over the keys, with and without a cap on
  the scores: prompts' portions and single tokens in one step, keys over page borders, first tokens, a request of one token.
  One key far back gets a score that stands out (its query and key are scaled), so a lost page or a wrong position shows."""
  from miniinfer_b200.kernels import ops
  items, nh, nkv, hd, page = ATTENTION_CASES[case]
  qkv, kv, bt, batch = make_attention_case(items, nh, nkv, hd, page, DT[dtype], seed=case, scale_q=0.5)
  bias = (-2.0 + torch.randn(nh, generator=torch.Generator().manual_seed(case))).to(DEV)
  scale = 1.0 / math.sqrt(hd)
  out = torch.zeros((qkv.shape[0], nh * hd), dtype=DT[dtype], device=DEV)
  ops.attention(out, qkv, kv, bt, batch, nh, nkv, hd, scale, None, softcap=softcap, score_bias=bias)
  want = plain_sigmoid_attention(qkv.cpu(), kv.cpu(), bt.cpu(), batch, nh, nkv, hd, scale, softcap, bias.cpu())
  bound = (2e-5 if dtype == "float32" else 1.5e-2) * float(want.abs().max())
  assert float((out.float().cpu() - want).abs().max()) <= bound
  if dtype == "bfloat16":      # the cap alone, under a softmax
    ops.attention(out, qkv, kv, bt, batch, nh, nkv, hd, scale, None, softcap=softcap)
    want = plain_sigmoid_attention(qkv.cpu(), kv.cpu(), bt.cpu(), batch, nh, nkv, hd, scale, softcap, bias.cpu(), sigmoid=False)
    assert float((out.float().cpu() - want).abs().max()) <= 1.5e-2 * float(want.abs().max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_stands_out_under_sigmoid_weights(dtype):
  """All weights but one are next to nothing (a bias of -20); one key 900 tokens back has a score of 29 for one head: the
  output of that head is that key's value, of the others nearly zero."""
  from miniinfer_b200.kernels import ops
  nh, nkv, hd, page = 4, 2, 64, 64
  for items in ([(1000, 1)], [(1000, 100)]):
    qkv, kv, bt, batch = make_attention_case(items, nh, nkv, hd, page, DT[dtype], seed=5, scale_q=0.05)
    slot = int(batch.seq_slot[0])
    far = 100
    key = kv[bt[slot, far // page].long(), 0, 1, far % page].float()
    qkv[-1, 3 * hd:4 * hd] = (key * (30.0 * math.sqrt(hd) / float(key.pow(2).sum()))).to(DT[dtype])      # head 3 reads kv head 1
    bias = torch.full((nh,), -20.0, device=DEV)
    out = torch.zeros((qkv.shape[0], nh * hd), dtype=DT[dtype], device=DEV)
    ops.attention(out, qkv, kv, bt, batch, nh, nkv, hd, 1.0 / math.sqrt(hd), None, softcap=100.0, score_bias=bias)
    value = kv[bt[slot, far // page].long(), 1, 1, far % page].float()
    got = out[-1].float().view(nh, hd)
    assert float((got[3] - value).abs().max()) <= 0.05 * float(value.abs().max()) + 0.05
    assert float(got[:3].abs().max()) <= 0.05
    want = plain_sigmoid_attention(qkv.cpu(), kv.cpu(), bt.cpu(), batch, nh, nkv, hd, 1.0 / math.sqrt(hd), 100.0, bias.cpu())
    assert float((out.float().cpu() - want).abs().max()) <= (2e-5 if dtype == "float32" else 1.5e-2) * float(want.abs().max())


def expert_weights(E, H, F, S, seed, dtype):
  g = torch.Generator().manual_seed(seed)
  W = {"router": torch.randn((E, H), generator=g) * 4.0 / math.sqrt(H), "shared.sg": torch.randn((1, H), generator=g) / math.sqrt(H),
       "shared.gate": torch.randn((S, H), generator=g) * 2.0 / math.sqrt(H), "shared.up": torch.randn((S, H), generator=g) * 2.0 / math.sqrt(H),
       "shared.down": torch.randn((H, S), generator=g) / math.sqrt(S)}
  for e in range(E):
    W[f"e{e}.gate"] = torch.randn((F, H), generator=g) * 2.0 / math.sqrt(H)
    W[f"e{e}.up"] = torch.randn((F, H), generator=g) * 2.0 / math.sqrt(H)
    W[f"e{e}.down"] = torch.randn((H, F), generator=g) / math.sqrt(F)
  return {k: rounded(v, dtype) for k, v in W.items()}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,E,top,H,F,S", [(1, 5, 2, 64, 24, 16), (7, 3, 3, 32, 16, 8), (70, 4, 1, 64, 40, 24), (700, 4, 2, 128, 64, 96),
                                            (1800, 6, 2, 64, 64, 64)])
def test_clamped_experts_with_a_gated_shared_expert(dtype, T, E, top, H, F, S):
  """The largest logits choose, the softmax over the chosen logits weighs, the clamps bite (limits of 0.7 and 0.5 against
  gate and up values of size 2), the shared expert comes in under its sigmoid: few rows, many rows (the tcgen05 grouped
  product in bfloat16), all experts chosen, one chosen."""
  from miniinfer_b200.engine.context import Workspace
  from miniinfer_b200.kernels import ops
  W = expert_weights(E, H, F, S, T + E, dtype)
  x = rounded(torch.randn((T, H), generator=torch.Generator().manual_seed(T)), dtype)
  mlp = plain.moe(F, 0.7, E, top, (S, 0.5))
  want = plain.mixture(x.double(), {("m." + k): v.double() for k, v in W.items()}, "m.", mlp).float()
  z = x.double() @ W["router"].double().T
  srt = torch.sort(z, dim=-1, descending=True).values
  clear = (srt[:, top - 1] - srt[:, top]) > (1e-4 if dtype == "float32" else 0.05) if top < E else torch.ones(T, dtype=torch.bool)
  dev = lambda t: t.to(DT[dtype]).to(DEV)
  ws = Workspace(torch.device(DEV)) if DEV != "cpu" else Workspace("cpu")
  router = dev(torch.cat((W["router"], W["shared.sg"])))
  gate_up = dev(torch.stack([torch.cat((W[f"e{e}.gate"], W[f"e{e}.up"])) for e in range(E)]))
  down = dev(torch.stack([W[f"e{e}.down"] for e in range(E)]))
  act = torch.zeros((T, S), dtype=DT[dtype], device=DEV)
  ops.linear_glu(act, dev(x), dev(torch.cat((W["shared.gate"], W["shared.up"]))), ws, "clamped", 0.5)
  g, u = x.double() @ W["shared.gate"].double().T, x.double() @ W["shared.up"].double().T
  g, u = g.clamp(max=0.5), u.clamp(-0.5, 0.5)
  want_act = (g * torch.sigmoid(1.702 * g) * (u + 1)).float()
  assert float((act.float().cpu() - want_act).abs().max()) <= (2e-5 if dtype == "float32" else 2e-2) * float(want_act.abs().max())
  shared = torch.zeros((T, H), dtype=DT[dtype], device=DEV)
  ops.linear(shared, act, dev(W["shared.down"]))
  out = torch.zeros((T, H), dtype=DT[dtype], device=DEV)
  ops.routed_experts(out, dev(x), router, None, gate_up, down, top, ws, weights="softmax_chosen", glu="clamped", limit=0.7,
                     shared=shared, shared_gated=True)
  diff = (out.float().cpu() - want).abs().max(-1).values
  assert int(clear.sum()) >= 0.8 * T
  assert float(diff[clear].max()) <= (3e-5 if dtype == "float32" else 4e-2) * float(want.abs().max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("M,parts,K,N", [(1, 3, 16, 32), (9, 1, 8, 16), (40, 5, 24, 48), (300, 2, 64, 128)])
def test_a_block_diagonal_map_part_by_part(dtype, M, parts, K, N):
  """out[b] = x[:, part b] @ w[b]^T: few rows (the batched kernels) and many (one strided batched library product)."""
  from miniinfer_b200.kernels import ops
  g = torch.Generator().manual_seed(M + parts)
  x, w = rounded(torch.randn((M, parts * K), generator=g), dtype), rounded(torch.randn((parts, N, K), generator=g), dtype)
  want = torch.einsum("mbk,bnk->bmn", x.double().view(M, parts, K), w.double()).float()
  out = torch.zeros((parts, M, N), dtype=torch.float32, device=DEV)
  ops.linear_parts(out, x.to(DT[dtype]).to(DEV), w.to(DT[dtype]).to(DEV))
  assert float((out.cpu() - want).abs().max()) <= 2e-5 * float(want.abs().max())


@pytest.mark.skipif(DEV == "cpu", reason="two forms of the CUDA kernel")
@pytest.mark.parametrize("softcap", [0.0, 6.0])
def test_sigmoid_weights_with_blocks_in_pairs(softcap, monkeypatch):
  """The tcgen05 prefill kernel with two blocks on a work (what steps of thousands of new tokens take) on shaped scores:
  the rows of blocks that work alone, and the plain sums."""
  from miniinfer_b200.kernels import ops
  nh, nkv, hd, page = 8, 2, 128, 64
  qkv, kv, bt, batch = make_attention_case([(400, 400), (129, 2), (64, 1)], nh, nkv, hd, page, torch.bfloat16, seed=9, scale_q=0.5)
  bias = (-2.0 + torch.randn(nh, generator=torch.Generator().manual_seed(2))).to(DEV)
  outs = []
  for pairs in ("1", "0"):
    monkeypatch.setenv("MINIINFER_B200_PREFILL_PAIRS", pairs)
    out = torch.zeros((qkv.shape[0], nh * hd), dtype=torch.bfloat16, device=DEV)
    ops.attention(out, qkv, kv, bt, batch, nh, nkv, hd, hd ** -0.5, None, softcap=softcap, score_bias=bias)
    outs.append(out.float().cpu())
  want = plain_sigmoid_attention(qkv.cpu(), kv.cpu(), bt.cpu(), batch, nh, nkv, hd, hd ** -0.5, softcap, bias.cpu())
  for o in outs:
    assert float((o - want).abs().max()) <= 1.5e-2 * float(want.abs().max())
  assert float((outs[0] - outs[1]).abs().max()) <= 4e-3 * float(want.abs().max())
