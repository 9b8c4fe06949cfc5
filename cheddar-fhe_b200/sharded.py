"""One HMult (tensor product, relinearisation, ModDown; no rescale) with the RNS
limbs of every polynomial sharded across the GPUs of one box.

Rank r of G owns the limbs whose position in the extended basis (the level's Q
limbs followed by the auxiliary limbs) is congruent to r modulo G, for the
ciphertexts, the evaluation key and the result alike. Element-wise work and
the transforms never leave a limb, so they need no communication. The two base
conversions do: a converted limb depends on every source limb of its digit.
The exchange is an all-gather of the small side of each conversion,

  * the inverse-transformed, pre-scaled limbs of d2 before ModUp
    (nq limbs in total, 256 KiB each), and
  * the inverse-transformed auxiliary limbs of the two accumulators before
    ModDown (2 * alpha limbs),

after which every rank converts into the destination limbs it owns. The
reference is single-GPU (include/core/DeviceVector.h:88); this follows the
algebra of its key switch (src/core/ModSwitch.cu:429-684,
src/core/Context.cpp:584-737) limb by limb, so the words are those of
cfhe_hmult(..., rescale = 0) on one GPU.

Everything here calls the C ABI through `Engine`; the collectives are
torch.distributed all_gather calls on device tensors (NCCL on GPUs; the
partition logic alone runs on gloo for the CPU test).
"""
import numpy as np


class LimbShardPlan:
    """Who owns which limb, and which limbs each digit's conversion reads and writes."""

    def __init__(self, params, level, world):
        self.p = params
        self.level = level
        self.world = world
        T, M = len(params["terminal_primes"]), len(params["main_primes"])
        self.alpha = len(params["auxiliary_primes"])
        nm, nt = params["level_config"][level]
        self.T, self.L = T, T + M
        self.q_g = list(range(T - nt, T + nm))                      # global prime indices of the Q limbs
        self.aux_g = [self.L + a for a in range(self.alpha)]
        self.full_g = self.q_g + self.aux_g
        self.nq, self.ntot = len(self.q_g), len(self.q_g) + self.alpha
        # digits: alpha-sized windows of the Q limbs, padded by the absent terminal slots
        off = T - nt
        padded = self.nq + off
        beta = (nm + T + self.alpha - 1) // self.alpha
        self.digits = []  # (digit number, first position, one past the last position)
        for i in range(beta):
            s0, s1 = i * self.alpha, min((i + 1) * self.alpha, padded)
            if s1 <= off:
                continue
            self.digits.append((i, max(0, s0 - off), s1 - off))
        self.primes = ([int(x) for x in reversed(params["terminal_primes"])] + [int(x) for x in params["main_primes"]] +
                       [int(x) for x in params["auxiliary_primes"]])

    def owner(self, pos):
        return pos % self.world

    def owned(self, rank):
        """Positions in the extended basis that `rank` owns."""
        return [k for k in range(self.ntot) if self.owner(k) == rank]

    def owned_q(self, rank):
        return [k for k in self.owned(rank) if k < self.nq]

    def owned_aux(self, rank):
        return [k for k in self.owned(rank) if k >= self.nq]

    def q(self, pos):
        return self.primes[self.full_g[pos]]

    def max_owned(self, positions):
        """Largest number of the given positions any rank owns (all-gather pads to it)."""
        return max(sum(1 for k in positions if self.owner(k) == r) for r in range(self.world))

    def modup_prescale(self, digit):
        """(S_hat_k * N)^-1 mod s_k for the source limbs of a digit (reference
        src/core/ModSwitch.cu:320-360)."""
        _, s0, s1 = digit
        n = 1 << self.p["log_degree"]
        out = {}
        for k in range(s0, s1):
            sk = self.q(k)
            v = n % sk
            for i in range(s0, s1):
                if i != k:
                    v = v * (self.q(i) % sk) % sk
            out[k] = pow(v, -1, sk)
        return out

    def moddown_prescale(self):
        n = 1 << self.p["log_degree"]
        out = {}
        for k in range(self.nq, self.ntot):
            pk = self.q(k)
            v = n % pk
            for i in range(self.nq, self.ntot):
                if i != k:
                    v = v * (self.q(i) % pk) % pk
            out[k] = pow(v, -1, pk)
        return out

    def p_mod(self, pos):
        """P = product of the auxiliary primes, modulo the prime at `pos`."""
        q, v = self.q(pos), 1
        for a in range(self.nq, self.ntot):
            v = v * (self.q(a) % q) % q
        return v


def _mont(x, q):
    return (int(x) << 32) % int(q)


def gather_limbs(dist, torch, local, positions, plan, rank, events=None):
    """All-gather of limb buffers: `local` holds this rank's limbs of
    `positions` (in order); returns one tensor [len(positions)][N] with the
    limbs of all ranks in the order of `positions` (one all-gather, one row
    selection). `events`: list that receives a (start, end) CUDA event pair
    around the collective."""
    mine = [k for k in positions if plan.owner(k) == rank]
    width = plan.max_owned(positions)
    n = local.shape[-1]
    if len(mine) == width:
        pad = local.contiguous()
    else:
        pad = torch.zeros((width, n), dtype=local.dtype, device=local.device)
        if mine:
            pad[:len(mine)] = local
    allbuf = torch.empty((plan.world, width, n), dtype=local.dtype, device=local.device)
    timed = events is not None and pad.is_cuda
    if timed:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    if plan.world > 1:
        dist.all_gather_into_tensor(allbuf.view(plan.world * width, n), pad)
    else:
        allbuf[0] = pad
    if timed:
        e1.record()
        events.append((e0, e1))
    # row of position k inside the gathered buffer: owner * width + its rank among the owner's positions
    seen = [0] * plan.world
    rows = []
    for k in positions:
        r = plan.owner(k)
        rows.append(r * width + seen[r])
        seen[r] += 1
    idx = torch.tensor(rows, dtype=torch.long, device=local.device)
    return allbuf.view(plan.world * width, n).index_select(0, idx)


def sharded_hmult(eng, plan, rank, dist, b1, a1, b2, a2, kb, ka):
    """b1..a2: this rank's Q limbs of the two ciphertexts, [owned_q][N]; kb, ka:
    this rank's limbs of the key digits, lists of [owned][N] (positions of the
    extended basis at this level). Returns this rank's Q limbs of (out_b, out_a)
    and the seconds spent inside the two collectives (device-timed)."""
    torch = eng.torch
    n = eng.n
    own = plan.owned(rank)
    own_q, own_aux = plan.owned_q(rank), plan.owned_aux(rank)
    gq = [plan.full_g[k] for k in own_q]
    g_own = [plan.full_g[k] for k in own]
    events = []
    # 1. tensor product on the owned Q limbs
    d0, d1, d2 = eng.empty(len(own_q), n), eng.empty(len(own_q), n), eng.empty(len(own_q), n)
    eng.tensor_(d0, d1, d2, b1, a1, b2, a2, gq)
    # 2. ModUp of d2: inverse transform with the digit's pre-scale constants, centred
    pre = {}
    for dg in plan.digits:
        pre.update(plan.modup_prescale(dg))
    y_own = eng.empty(len(own_q), n)
    eng.intt_(y_own, d2, gq, consts=[pre[k] for k in own_q], centred=True)
    y_all = gather_limbs(dist, torch, y_own, list(range(plan.nq)), plan, rank, events)  # [nq][N]
    # per digit: the owned limbs outside the digit are converted and transformed
    # straight into their rows, the owned limbs inside it are d2 itself
    dev = d2.device
    mu = []
    for (_, s0, s1) in plan.digits:
        src = y_all[s0:s1]
        src_g = [plan.full_g[k] for k in range(s0, s1)]
        buf = eng.empty(len(own), n)
        outside = [i for i, k in enumerate(own) if k < s0 or k >= s1]
        inside = [i for i, k in enumerate(own) if s0 <= k < s1]
        if outside:
            dst_g = [plan.full_g[own[i]] for i in outside]
            conv = eng.empty(len(outside), n)
            eng.bconv_(conv, src, src_g, dst_g)
            eng.ntt_(conv, conv, dst_g)
            buf.index_copy_(0, torch.tensor(outside, dtype=torch.long, device=dev), conv)
        if inside:
            rows = torch.tensor([own_q.index(own[i]) for i in inside], dtype=torch.long, device=dev)
            buf.index_copy_(0, torch.tensor(inside, dtype=torch.long, device=dev), d2.index_select(0, rows))
        mu.append(buf)
    # 3. inner product with the key on the owned limbs, plus P * (d0, d1) on the Q limbs
    pm = [_mont(plan.p_mod(k), plan.q(k)) for k in own_q]
    acc = []
    for part, key, d in ((0, kb, d0), (1, ka, d1)):
        add = torch.zeros((len(own), n), dtype=torch.int32, device=d.device)
        if own_q:
            eng.const_op_(3, add[:len(own_q)], d, None, pm, gq)
        out = eng.empty(len(own), n)
        eng.nary_("plain", [out], [[m] for m in mu], g_own, pts=key, addend=[add])
        acc.append(out)
    # 4. ModDown: inverse transform of the owned auxiliary limbs, gather, convert, transform, (x - t) / P
    pre_d = plan.moddown_prescale()
    aux_pos = list(range(plan.nq, plan.ntot))
    g_aux = [plan.full_g[k] for k in own_aux]
    outs = []
    gathered = []
    for part in range(2):
        z = eng.empty(len(own_aux), n)
        if own_aux:
            eng.intt_(z, acc[part][len(own_q):], g_aux, consts=[pre_d[k] for k in own_aux], centred=True)
        gathered.append(gather_limbs(dist, torch, z, aux_pos, plan, rank, events))  # [alpha][N]
    pinv = [_mont(pow(plan.p_mod(k), -1, plan.q(k)), plan.q(k)) for k in own_q]
    for part in range(2):
        src = gathered[part]
        t = eng.empty(len(own_q), n)
        res = eng.empty(len(own_q), n)
        if own_q:
            eng.bconv_(t, src, [plan.full_g[k] for k in aux_pos], gq)
            eng.ntt_(t, t, gq)
            eng.binary_(1, res, acc[part][:len(own_q)], t, gq)
            eng.const_op_(3, res, res, None, pinv, gq)
        outs.append(res)
    seconds = 0.0
    if events:
        torch.cuda.synchronize()
        seconds = sum(a.elapsed_time(b) for a, b in events) * 1e-3
    return outs[0], outs[1], seconds
