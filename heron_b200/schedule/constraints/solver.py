"""A small finite-domain constraint solver behind the reference's ``Solver`` interface
(schedule/constraints/ortools/solver.py:17-177): ``solve(hint, known, bounds)``,
``validate(knob_dict)``, ``repair(val_dict)``, ``SATScore`` / ``MultiSATScore`` and ``dump``.

The reference builds an OR-tools CP-SAT model per call.  OR-tools is a third-party dependency
this build does not have; the knob spaces here are small (tens of variables, small candidate
sets), so interval propagation plus randomised depth-first search is enough:

* every variable has an integer interval [low, up];
* propagation narrows intervals through the primitives until nothing changes
  (EQ/LE/LT/NE, ProdTwo and Sum over non-negative integers, optional 0/1 condition);
* search assigns the still-open variables one at a time — hinted value first, the rest of the
  (small) domain in random order — propagating after each assignment and backtracking on a
  wipe-out.  Variable and value order are shuffled per call, which is what gives
  ``KnobManager.randSample`` its diversity (the reference shuffles variables, constraints and
  hints for the same reason, solver.py:124-160).
"""
import random

from .primitives import EQ, LE, LT, NE, ProdTwo, Sum


class Variable:
    def __init__(self, name, low, up, item, defv):
        self.low = low
        self.up = up
        self.item = item
        self.defv = defv
        self.name = name

    def __repr__(self):
        return "Var(%s, %d, %d, %d)" % (self.name, self.low, self.up, self.defv)


class _Wipeout(Exception):
    pass


def _ceil_div(a, b):
    return -((-a) // b)


class _State:
    """Intervals of one search node; copy-on-branch."""

    __slots__ = ("lo", "hi")

    def __init__(self, lo, hi):
        self.lo = lo
        self.hi = hi

    def copy(self):
        return _State(dict(self.lo), dict(self.hi))

    def bounds(self, v):
        if isinstance(v, str):
            return self.lo[v], self.hi[v]
        return v, v

    def narrow(self, v, lo, hi):
        """Intersects v's interval with [lo, hi]; returns True when it changed."""
        if not isinstance(v, str):
            if lo > v or hi < v:
                raise _Wipeout()
            return False
        clo, chi = self.lo[v], self.hi[v]
        nlo, nhi = max(clo, lo), min(chi, hi)
        if nlo > nhi:
            raise _Wipeout()
        if nlo != clo or nhi != chi:
            self.lo[v], self.hi[v] = nlo, nhi
            return True
        return False


def _prop_binary(p, st):
    """Propagates one EQ/LE/LT/NE; returns True when some interval changed."""
    a, b = p.args
    if p.cond is not None:
        clo, chi = st.bounds(p.cond)
        if chi == 0:
            return False
        if clo == 0:
            # Condition open: if the relation cannot hold, the condition must be 0.
            alo, ahi = st.bounds(a)
            blo, bhi = st.bounds(b)
            impossible = (
                (isinstance(p, EQ) and (ahi < blo or bhi < alo))
                or (isinstance(p, LE) and alo > bhi)
                or (isinstance(p, LT) and alo >= bhi)
                or (isinstance(p, NE) and alo == ahi == blo == bhi)
            )
            return st.narrow(p.cond, 0, 0) if impossible else False
    alo, ahi = st.bounds(a)
    blo, bhi = st.bounds(b)
    ch = False
    if isinstance(p, EQ):
        ch |= st.narrow(a, blo, bhi)
        alo, ahi = st.bounds(a)
        ch |= st.narrow(b, alo, ahi)
    elif isinstance(p, LE):
        ch |= st.narrow(a, alo, bhi)
        ch |= st.narrow(b, alo, bhi)
    elif isinstance(p, LT):
        ch |= st.narrow(a, alo, bhi - 1)
        ch |= st.narrow(b, alo + 1, bhi)
    elif isinstance(p, NE):
        if alo == ahi and blo == bhi and alo == blo:
            raise _Wipeout()
        if alo == ahi and isinstance(b, str):
            if blo == alo:
                ch |= st.narrow(b, blo + 1, bhi)
            elif bhi == alo:
                ch |= st.narrow(b, blo, bhi - 1)
        if blo == bhi and isinstance(a, str):
            if alo == blo:
                ch |= st.narrow(a, alo + 1, ahi)
            elif ahi == blo:
                ch |= st.narrow(a, alo, ahi - 1)
    return ch


def _prop_prod(p, st):
    t, (a, b) = p.args
    alo, ahi = st.bounds(a)
    blo, bhi = st.bounds(b)
    if alo < 0 or blo < 0:
        raise ValueError("ProdTwo over negative domains is not supported")
    ch = st.narrow(t, alo * blo, ahi * bhi)
    tlo, thi = st.bounds(t)
    if bhi > 0 and blo > 0:
        ch |= st.narrow(a, _ceil_div(tlo, bhi), thi // blo)
    alo, ahi = st.bounds(a)
    if ahi > 0 and alo > 0:
        ch |= st.narrow(b, _ceil_div(tlo, ahi), thi // alo)
    # With both factors fixed the target is fixed; with target and one factor fixed, divisibility.
    alo, ahi = st.bounds(a)
    blo, bhi = st.bounds(b)
    tlo, thi = st.bounds(t)
    if tlo == thi:
        for x, (ylo, yhi) in ((a, (blo, bhi)), (b, (alo, ahi))):
            if ylo == yhi and ylo > 0:
                if tlo % ylo != 0:
                    raise _Wipeout()
                ch |= st.narrow(x, tlo // ylo, tlo // ylo)
    return ch


def _prop_sum(p, st):
    t, terms = p.args
    los = [st.bounds(x)[0] for x in terms]
    his = [st.bounds(x)[1] for x in terms]
    slo, shi = sum(los), sum(his)
    ch = st.narrow(t, slo, shi)
    tlo, thi = st.bounds(t)
    for x, lo, hi in zip(terms, los, his):
        ch |= st.narrow(x, tlo - (shi - hi), thi - (slo - lo))
    return ch


def _propagate(primitives, st, watch=None):
    """Runs every primitive to a fixpoint (the models are small; no queue bookkeeping needed)."""
    changed = True
    while changed:
        changed = False
        for p in primitives:
            if isinstance(p, ProdTwo):
                changed |= _prop_prod(p, st)
            elif isinstance(p, Sum):
                changed |= _prop_sum(p, st)
            else:
                changed |= _prop_binary(p, st)


class Solver:
    # Upper limit on search nodes per solve; the knob spaces need a few hundred at most.
    node_limit = 200000
    # Variables whose interval is wider than this are never branched on before narrower ones.
    enum_limit = 4096

    def __init__(self):
        self.vals = {}
        self.primitives = []

    def addVal(self, name, low, up, def_val):
        assert name not in self.vals
        self.vals[name] = Variable(name, low, up, None, def_val)

    def getVal(self, v):
        if isinstance(v, str):
            assert v in self.vals
            return self.vals[v].item
        if isinstance(v, int):
            return v
        raise TypeError(v)

    # -- search ------------------------------------------------------------------------------
    def _initial(self, bounds=None, fixed=None):
        lo, hi = {}, {}
        for k, v in self.vals.items():
            l, u = v.low, v.up
            if bounds and k in bounds:
                l, u = max(l, bounds[k][0]), min(u, bounds[k][1])
            if fixed and k in fixed:
                l = u = fixed[k]
            lo[k], hi[k] = l, u
        return _State(lo, hi)

    def _search(self, st, prims, hint, pairs, rng, randomize):
        nodes = [0]
        order = list(self.vals.keys())
        if randomize:
            rng.shuffle(order)

        def pick(state):
            best, best_w = None, None
            for k in order:
                w = state.hi[k] - state.lo[k]
                if w == 0:
                    continue
                if best is None or w < best_w:
                    best, best_w = k, w
                    if w == 1:
                        break
            return best

        def values(state, k):
            lo, hi = state.lo[k], state.hi[k]
            if k in pairs:
                cands = [c for c in pairs[k] if lo <= c <= hi]
            elif hi - lo + 1 <= self.enum_limit:
                cands = list(range(lo, hi + 1))
            else:
                # A wide derived variable that propagation has not fixed: probe its ends and
                # a few random interior points rather than the whole interval.
                cands = sorted({lo, hi} | {rng.randint(lo, hi) for _ in range(32)})
            if randomize:
                rng.shuffle(cands)
            if k in hint and hint[k] in cands:
                cands.remove(hint[k])
                cands.insert(0, hint[k])
            return cands

        def pairs_ok(state):
            # a two-valued `known` entry is a real two-element domain, not the interval between
            # its values: a state whose interval holds neither value is dead
            for k, cands in pairs.items():
                lo, hi = state.lo[k], state.hi[k]
                if not any(lo <= c <= hi for c in cands):
                    return False
            return True

        def rec(state):
            nodes[0] += 1
            if nodes[0] > self.node_limit:
                return None
            k = pick(state)
            if k is None:
                return state
            for c in values(state, k):
                child = state.copy()
                child.lo[k] = child.hi[k] = c
                try:
                    _propagate(prims, child)
                except _Wipeout:
                    continue
                if not pairs_ok(child):
                    continue
                res = rec(child)
                if res is not None:
                    return res
            return None

        try:
            _propagate(prims, st)
        except _Wipeout:
            return None
        if not pairs_ok(st):
            return None
        return rec(st)

    def _solve(self, hint=None, known=None, bounds=None, fixed=None, randomize=True):
        rng = random
        prims = list(self.primitives)
        if randomize:
            rng.shuffle(prims)
        st = self._initial(bounds, fixed)
        pairs = {}
        for key, cands in (known or {}).items():
            assert 1 <= len(cands) <= 2
            if len(cands) == 1:
                try:
                    st.narrow(key, cands[0], cands[0])
                except _Wipeout:
                    return False, None
            else:
                pairs[key] = sorted(set(cands))
                try:
                    st.narrow(key, pairs[key][0], pairs[key][-1])
                except _Wipeout:
                    return False, None
        res = self._search(st, prims, hint or {}, pairs, rng, randomize)
        if res is None:
            return False, None
        out = []
        for k in self.vals:
            self.vals[k].item = res.lo[k]
            out.append(res.lo[k])
        return True, out

    # -- the reference's entry points --------------------------------------------------------
    def solve(self, hint, known, bounds={}):
        """A random feasible point: ``hint`` values are tried first, ``known`` maps a variable
        to one forced value or to two allowed values (constrained crossover), ``bounds`` to an
        interval (solver.py:120-177)."""
        return self._solve(hint=hint, known=known, bounds=bounds, randomize=True)

    def validate(self, knob_dict):
        """Is there a feasible completion with these variables fixed? (solver.py:35-58)"""
        for k, v in knob_dict.items():
            var = self.vals.get(k)
            if var is None or v < var.low or v > var.up:
                return False, None
        return self._solve(fixed=knob_dict, randomize=False)

    def repair(self, val_dict):
        """A feasible point as close to ``val_dict`` as the hinted search gets (solver.py:91-118)."""
        return self._solve(hint=val_dict, randomize=False)

    def SATScore(self, val_dict):
        return sum(p.eval(val_dict) for p in self.primitives)

    def MultiSATScore(self, val_dict):
        scores = [p.eval(val_dict) for p in self.primitives]
        return scores, all(s == 0 for s in scores)

    def dump(self):
        """The model as text: one line per variable and per primitive (written to constraints.py
        by Task.dump_constraints, as the reference does at task/task.py:70-74)."""
        lines = ["# finite-domain model: variables then constraints"]
        for k, v in self.vals.items():
            lines.append("var %s in [%d, %d] default %d" % (k, v.low, v.up, v.defv))
        for p in self.primitives:
            lines.append(p.desc())
        return "\n".join(lines) + "\n"
