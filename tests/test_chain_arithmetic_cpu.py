"""The arithmetic behind `cta_chain` (scriptonait_b200/csrc/sampler_device.cuh), stated in Python and checked
against plain sequential float32 arithmetic: inside one binade a running f32 value is an integer A times
its ulp, a rounded addition or subtraction of a term is an integer step that depends on A only through its
parity (and only when the term falls exactly between two floats), and whatever leaves the binade, reaches
the top-p bound or ends the walk is an "event" whose term is evaluated with real float arithmetic. The
chains are the reference's: the softmax denominator (generate.rs:374), the cumulative probability up to
top_p (:397-409) and the draw's walk (:413-418). The second half checks that the same integers come out of
an associative composition of two-state machines, which is what lets the GPU use a prefix scan."""
import numpy as np

f32 = np.float32

def decode(x):
    b = int(np.float32(x).view(np.uint32))
    e = (b >> 23) & 0xff
    m = b & 0x7fffff
    if e == 0:
        return m, -126          # subnormal or zero: value = m * 2^(-126-23)
    return m | 0x800000, e - 127  # value = M * 2^(E-23)

def chunk_add(v, pos, C, s, bound_val):
    """One chunk attempt. s: f32 normal > 0. Returns (event_index or None, A_before_event or A_end, es)."""
    Ms, es = decode(s)
    A = Ms
    # bound: first i whose state after the element reaches min(2^24, T)
    B = 1 << 24
    if bound_val is not None:
        Mt, Et = decode(bound_val)
        if Et < es: B = 0            # every state qualifies
        elif Et == es: B = min(B, Mt)
    for i in range(pos, min(pos + C, len(v))):
        M, E = decode(v[i])
        shift = es - E
        if shift < 0:
            return i, A, es          # element above the state's binade: handle with real arithmetic
        if shift >= 32: fl, rem, half = 0, M, 1 << 40
        else:
            fl = M >> shift
            rem = M & ((1 << shift) - 1)
            half = (1 << (shift - 1)) if shift >= 1 else (1 << 40)
        if shift == 0: c = 0
        elif rem > half: c = 1
        elif rem < half: c = 0
        else: c = (A + fl) & 1
        A2 = A + fl + c
        if A2 >= B:
            return i, A, es
        A = A2
    return None, A, es

def state(A, es):
    return f32(np.ldexp(np.float64(A), es - 23))

def chain_add(v, s0, C=64, top_p=None):
    v = np.asarray(v, f32); n = len(v); s = f32(s0); pos = 0
    while pos < n:
        Ms, es = decode(s)
        if not (s > 0 and ((int(s.view(np.uint32)) >> 23) & 0xff) != 0):   # zero / subnormal state: real arithmetic
            s = f32(s + v[pos]); 
            if top_p is not None and s >= top_p: return pos, s
            pos += 1; continue
        ev, A, es = chunk_add(v, pos, C, s, top_p)
        if ev is None:
            s = state(A, es); pos = min(pos + C, n); continue
        s = f32(state(A, es) + v[ev])
        if top_p is not None and s >= top_p: return ev, s
        pos = ev + 1
    return n, s

def chunk_sub(v, pos, C, r):
    Mr, es = decode(r)
    A = Mr
    for i in range(pos, min(pos + C, len(v))):
        M, E = decode(v[i])
        shift = es - E
        if shift < 0: return i, A, es
        if shift >= 32: fl, rem, half = 0, M, 1 << 40
        else:
            fl = M >> shift
            rem = M & ((1 << shift) - 1)
            half = (1 << (shift - 1)) if shift >= 1 else (1 << 40)
        if A - fl - (1 if rem > 0 else 0) < (1 << 23):
            return i, A, es          # hit, or the result leaves the binade: real arithmetic
        if shift == 0: c = 0
        elif rem > half: c = 1
        elif rem < half: c = 0
        else: c = (A - fl) & 1
        A = A - fl - c
    return None, A, es

def chain_walk(v, r0, C=64):
    v = np.asarray(v, f32); n = len(v); r = f32(r0); pos = 0
    while pos < n:
        if not (r > 0 and ((int(r.view(np.uint32)) >> 23) & 0xff) != 0):
            if r < v[pos]: return pos, r
            r = f32(r - v[pos]); pos += 1; continue
        ev, A, es = chunk_sub(v, pos, C, r)
        if ev is None:
            r = state(A, es); pos = min(pos + C, n); continue
        rb = state(A, es)
        if rb < v[ev]: return ev, rb
        r = f32(rb - v[ev]); pos = ev + 1
    return n, r

def seq_add(v, s0, top_p=None):
    s = f32(s0)
    for i, x in enumerate(np.asarray(v, f32)):
        s = f32(s + x)
        if top_p is not None and s >= top_p: return i, s
    return len(v), s

def seq_walk(v, r0):
    r = f32(r0)
    for i, x in enumerate(np.asarray(v, f32)):
        if r < x: return i, r
        r = f32(r - x)
    return len(v), r



def _descending_exponentials(g, n, kind):
    if kind == 0: x = g.normal(0, 1, n)
    elif kind == 1: x = g.normal(0, 5, n)
    elif kind == 2: x = np.round(g.normal(0, 2, n) * 4) / 4          # many equal values
    elif kind == 3: x = g.normal(0, 0.01, n)
    elif kind == 4: x = np.zeros(n)
    else: x = g.integers(-20, 3, n).astype(np.float64) * np.log(2)   # near powers of two
    x = np.sort(x.astype(np.float32))[::-1]
    return np.exp((x - x[0]).astype(np.float64)).astype(np.float32)


def _same(a, b):
    return a[0] == b[0] and np.float32(a[1]).view(np.uint32) == np.float32(b[1]).view(np.uint32)


def test_chunked_integer_chains_equal_sequential_float32():
    g = np.random.default_rng(11)
    for trial in range(90):
        n = int(g.integers(1, 1200))
        e = _descending_exponentials(g, n, trial % 6)
        chunk = int(g.choice([8, 64, 256]))
        total = seq_add(e, 0.0)
        assert _same(total, chain_add(e, 0.0, C=chunk)), ("sum", trial)
        p = (e / total[1]).astype(np.float32)
        top_p = f32(g.choice([0.5, 0.9, 0.95, 0.999, 0.3333]))
        cut = seq_add(p, 0.0, top_p)
        assert _same(cut, chain_add(p, 0.0, C=chunk, top_p=top_p)), ("cumulative", trial)
        keep = min(cut[0] + 1, n)
        u = f32(g.random())
        assert seq_walk(p[:keep], f32(u * cut[1]))[0] == chain_walk(p[:keep], f32(u * cut[1]), C=chunk)[0], ("walk", trial)
        assert seq_walk(e, f32(u * total[1]))[0] == chain_walk(e, f32(u * total[1]), C=64)[0], ("long walk", trial)


def test_exact_halves_follow_the_parity_of_the_running_value():
    # 2^24 - 2 is even, 2^24 - 1 odd at ulp 1... one binade lower: value 2^23 + k at ulp 1, terms of exactly 0.5
    for start in (8388608.0, 8388609.0, 12582911.0):
        v = np.full(50, 0.5, np.float32)
        assert _same(seq_add(v, f32(start)), chain_add(v, f32(start), C=8))
        assert seq_walk(v, f32(start))[1] == chain_walk(v, f32(start), C=8)[1]

def elem_trans(fl, gt, tie):
    inc = [0, 0]; par = [0, 0]
    for p in (0, 1):
        d = fl + (((p + fl) & 1) if tie else gt)
        inc[p] = d; par[p] = (p + d) & 1
    return inc, par
def compose(f, g):
    inc = [f[0][p] + g[0][f[1][p]] for p in (0, 1)]
    par = [g[1][f[1][p]] for p in (0, 1)]
    return inc, par


def test_machines_compose_associatively_to_the_sequential_integers():
    g = np.random.default_rng(3)
    for _ in range(200):
        n = int(g.integers(1, 200)); A0 = int(g.integers(1 << 23, 1 << 24))
        els = [(int(g.integers(0, 50)), int(g.integers(0, 2)), int(g.integers(0, 4) == 0)) for _ in range(n)]
        A = A0; seq = []
        for fl, gt, tie in els:
            A += fl + (((A + fl) & 1) if tie else gt); seq.append(A)
        ts = [elem_trans(*e) for e in els]
        acc = ([0, 0], [0, 1]); out = []
        for t in ts:
            acc = compose(acc, t); out.append(A0 + acc[0][A0 & 1])
        assert out == seq

        def tree(lo, hi):
            if hi - lo == 1: return ts[lo]
            mid = (lo + hi) // 2
            return compose(tree(lo, mid), tree(mid, hi))
        tot = tree(0, n)
        assert A0 + tot[0][A0 & 1] == seq[-1]
