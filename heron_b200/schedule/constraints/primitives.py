"""Constraint primitives of the knob space, with the reference's names, argument conventions and
violation scores (schedule/constraints/ortools/primitives.py:13-180).

Where the reference hands each primitive to OR-tools CP-SAT, these objects describe themselves
to the in-repo finite-domain solver (solver.py): ``propagate`` narrows variable intervals and
``eval`` gives the violation used by the unconstrained GA variants.  A primitive may carry a
``cond`` variable (0/1): it is enforced only when ``cond`` is 1.
"""


def getVal(val_dict, v):
    if isinstance(v, str):
        assert v in val_dict, v
        return val_dict[v]
    if isinstance(v, int):
        return v
    raise TypeError(v)


class _Binary:
    op = "?"

    def __init__(self, args, cond=None):
        assert len(args) == 2
        self.args = args
        self.cond = cond

    def variables(self):
        vs = [a for a in self.args if isinstance(a, str)]
        if self.cond is not None:
            vs.append(self.cond)
        return vs

    def desc(self):
        s = "%s %s %s" % (self.args[0], self.op, self.args[1])
        return s + (" if %s" % self.cond if self.cond is not None else "")

    def _active(self, val_dict):
        return self.cond is None or getVal(val_dict, self.cond) == 1


class LE(_Binary):
    op = "<="

    def eval(self, val_dict):
        if not self._active(val_dict):
            return 0
        return max(getVal(val_dict, self.args[0]) - getVal(val_dict, self.args[1]), 0)


class LT(_Binary):
    op = "<"

    def eval(self, val_dict):
        if not self._active(val_dict):
            return 0
        return max(getVal(val_dict, self.args[0]) - getVal(val_dict, self.args[1]) + 1, 0)


class EQ(_Binary):
    op = "=="

    def eval(self, val_dict):
        if not self._active(val_dict):
            return 0
        return abs(getVal(val_dict, self.args[1]) - getVal(val_dict, self.args[0]))


class NE(_Binary):
    op = "!="

    def eval(self, val_dict):
        if not self._active(val_dict):
            return 0
        return 0 if getVal(val_dict, self.args[0]) != getVal(val_dict, self.args[1]) else 1


class ProdTwo:
    """args = [target, [a, b]]: target == a * b."""

    cond = None

    def __init__(self, args):
        assert len(args) == 2 and len(args[1]) == 2
        self.args = args

    def variables(self):
        return [v for v in [self.args[0]] + list(self.args[1]) if isinstance(v, str)]

    def desc(self):
        return "%s == %s * %s" % (self.args[0], self.args[1][0], self.args[1][1])

    def eval(self, val_dict):
        t = getVal(val_dict, self.args[0])
        return abs(t - getVal(val_dict, self.args[1][0]) * getVal(val_dict, self.args[1][1]))


class Sum:
    """args = [target, [terms...]]: target == sum(terms)."""

    cond = None

    def __init__(self, args):
        assert len(args) == 2
        self.args = args

    def variables(self):
        return [v for v in [self.args[0]] + list(self.args[1]) if isinstance(v, str)]

    def desc(self):
        return "%s == sum(%s)" % (self.args[0], ", ".join(str(x) for x in self.args[1]))

    def eval(self, val_dict):
        t = getVal(val_dict, self.args[0])
        return abs(t - sum(getVal(val_dict, x) for x in self.args[1]))
