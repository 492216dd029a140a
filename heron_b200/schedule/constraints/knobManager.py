"""KnobManager: the registry of tunable knobs, derived variables and constraints of one task,
with the reference's interface (schedule/constraints/ortools/knobManager.py:15-479).

Schedule rules call ``define_value`` / ``addProd`` / ``addSUM`` / ``addLE`` / ``addEQ`` /
``addCandidates`` / ``addSelect`` while ``is_building`` is true; tuners then draw feasible
points with ``randSample`` and recombine them with the crossover / walk operators below.  After
a point is chosen (``is_building`` false) ``get_val`` returns the solved value of a variable.
"""
import random

import numpy as np

from .primitives import EQ, LE, LT, NE, ProdTwo, Sum
from .solver import Solver


class KnobManager:
    def __init__(self):
        self.sched_tups = []
        self.is_building = True
        self.solver = Solver()

        self.axis_parents = {}
        self.axis_brother = {}
        self.axis_ori_lenth = {}
        self.mems = []
        self.staged_fused_axes = set()

        self.knob_names = []
        self.solved_knob_vals_genotype = {}
        self.solved_knob_vals_phenotype = {}
        self.candidates = {}
        self._valid = False

        self.constraint_descs = ""
        self.dump_descs = False
        self.sched_desc = ""
        self.runtime_perf = None

    # -- lookup ------------------------------------------------------------------------------
    def get_val(self, name):
        if isinstance(name, int):
            return name
        assert isinstance(name, str)
        if name in self.axis_ori_lenth and name not in self.staged_fused_axes:
            return self.axis_ori_lenth[name]
        if self.is_building:
            return self.solver.vals[name].defv
        return self.solved_knob_vals_phenotype.get(name)

    def get_ax(self, ax):
        if ax in self.solver.vals:
            return ax
        if ax in self.axis_ori_lenth and ax not in self.staged_fused_axes:
            return self.axis_ori_lenth[ax]
        raise KeyError(ax)

    # -- model building ----------------------------------------------------------------------
    def define_value(self, name, low, up, def_val, is_knob=False):
        if not self.is_building:
            return name
        if name in self.solver.vals:
            return name
        if is_knob:
            self.knob_names.append(name)
        self.solver.addVal(name, low, up, def_val)
        return name

    def _desc(self, s):
        if self.dump_descs:
            self.constraint_descs += s

    def addProd(self, src, res):
        if not self.is_building:
            return
        if len(src) == 1:
            self.solver.primitives.append(EQ([src[0], res]))
        elif len(src) == 2:
            self.solver.primitives.append(ProdTwo([res, [src[0], src[1]]]))
        else:
            a = src[0]
            up = self.solver.vals[res].up if isinstance(res, str) else res
            for i in range(len(src) - 2):
                temp = str(a) + "_" + str(src[i + 1])
                self.define_value(temp, 1, up, 1)
                self.solver.primitives.append(ProdTwo([temp, [a, src[i + 1]]]))
                a = temp
            self.solver.primitives.append(ProdTwo([res, [a, src[-1]]]))
        self._desc("&Prod(%s,%s)" % (res, list(src)))

    def addLE(self, a, b):
        if not self.is_building:
            return
        assert isinstance(a, str)
        if isinstance(b, str):
            self.solver.primitives.append(LE([a, b]))
        else:
            self.changeUp(a, b)
        self._desc("&LE(%s,%s)" % (a, b))

    def addEQ(self, a, b):
        if not self.is_building:
            return
        assert isinstance(a, str)
        if isinstance(b, str):
            self.solver.primitives.append(EQ([a, b]))
        else:
            self.changeUp(a, b)
            self.changeLow(a, b)
        self._desc("&EQ(%s,%s)" % (a, b))

    def addNE(self, a, b):
        if not self.is_building:
            return
        self.solver.primitives.append(NE([a, b]))
        self._desc("&NE(%s,%s)" % (a, b))

    def addLT(self, a, b):
        if not self.is_building:
            return
        assert isinstance(a, str)
        if isinstance(b, str):
            self.solver.primitives.append(LT([a, b]))
        else:
            self.changeUp(a, b - 1)
        self._desc("&LT(%s,%s)" % (a, b))

    def addSUM(self, resname, keys):
        if not self.is_building:
            return
        self.solver.primitives.append(Sum([resname, keys]))
        self._desc("&SUM(%s,%s)" % (resname, list(keys)))

    def addSelect(self, cand_keys, knob_key, val_key):
        """val_key == cand_keys[knob_key] through one-hot auxiliaries (knobManager.py:189-208)."""
        if not self.is_building:
            return
        up = min(len(cand_keys) - 1, self.solver.vals[knob_key].up)
        keys = []
        for i in range(up + 1):
            assert "P#" in knob_key
            key = (knob_key + "_select%d" % i).replace("P#", "O#")
            self.define_value(key, 0, 1, 0)
            self.solver.primitives.append(EQ([val_key, cand_keys[i]], cond=key))
            self.solver.primitives.append(EQ([knob_key, i], cond=key))
            keys.append(key)
        self.solver.primitives.append(Sum([1, keys]))
        self._desc("&SELECT(%s,%s,%s)" % (val_key, knob_key, list(cand_keys)))

    def addCandidates(self, valname, candidates):
        """valname IN candidates through one-hot auxiliaries (knobManager.py:219-240)."""
        if not self.is_building:
            return
        idxs = []
        for idx, _ in enumerate(candidates):
            idx_name = valname + "_cand%d" % idx
            idx_name = idx_name.replace("P#", "O#") if "P#" in valname else "O#" + idx_name
            self.define_value(idx_name, 0, 1, 0)
            self.solver.primitives.append(EQ([valname, candidates[idx]], cond=idx_name))
            idxs.append(idx_name)
        self.solver.primitives.append(Sum([1, idxs]))
        if valname in self.knob_names:
            self.candidates[valname] = list(candidates)
        self._desc("&IN(%s,%s)" % (valname, list(candidates)))

    def addRawCandidates(self, valname, candidates):
        if not self.is_building:
            return
        self.candidates[valname] = list(candidates)

    def changeUp(self, a, b):
        self.solver.vals[a].up = min(self.solver.vals[a].up, b)

    def changeLow(self, a, b):
        self.solver.vals[a].low = max(self.solver.vals[a].low, b)

    def get_knob_candidates(self, name):
        if name in self.candidates:
            return self.candidates[name]
        low, up = self.solver.vals[name].low, self.solver.vals[name].up
        assert up - low + 1 <= 30
        return list(range(low, up + 1))

    # -- sampling and genetic operators ------------------------------------------------------
    def _store(self, point):
        for idx, key in enumerate(list(self.solver.vals.keys())):
            self.solved_knob_vals_genotype[key] = point[idx]
            self.solved_knob_vals_phenotype[key] = point[idx]

    def randSample(self, known={}, bounds={}):
        hint = {}
        for key in self.knob_names:
            if key in known:
                continue
            candidates = self.get_knob_candidates(key)
            hint[key] = candidates[random.randint(0, len(candidates) - 1)]
        valid, point = self.solver.solve(hint=hint, known=known, bounds=bounds)
        assert valid
        self._valid = valid
        self._store(point)
        return valid, point

    def validate(self, knob_dict):
        valid, point = self.solver.validate(knob_dict)
        self._valid = valid
        if valid:
            self._store(point)
        else:
            for key in knob_dict:
                self.solved_knob_vals_genotype[key] = knob_dict[key]
                self.solved_knob_vals_phenotype[key] = knob_dict[key]
            point = [knob_dict[key] for key in knob_dict]
        return point, valid

    def constrained_crossover_and_mutate(self, m1, m2, keys):
        """CGA's operator: each key variable but one (the mutation) must take one of its two
        parents' values; the solver completes the rest (knobManager.py:326-339)."""
        known = {}
        if len(keys) > 0:
            midx = random.randint(0, len(keys) - 1)
            for idx, key in enumerate(keys):
                if idx == midx:
                    continue
                known[key] = [m1.solved_knob_vals_genotype[key], m2.solved_knob_vals_genotype[key]]
        try:
            valid, res = self.randSample(known)
        except AssertionError:
            # The two parents' values admit no joint completion: fall back to a free sample.
            valid, res = self.randSample({})
        return res, valid

    def onepoint_crossover_and_mutation(self, keys, m1, m2, feasible):
        position = random.randint(0, len(keys) - 1)
        m1_keys = keys[:position]
        known = {}
        mkey = keys[random.randint(0, len(keys) - 1)]
        res = []
        for key in m1.solved_knob_vals_genotype.keys():
            if key == mkey:
                cands = feasible[key]
                known[key] = cands[random.randint(0, len(cands) - 1)]
            elif key in m1_keys:
                known[key] = m1.solved_knob_vals_genotype[key]
            else:
                known[key] = m2.solved_knob_vals_genotype[key]
            res.append(known[key])
        return known, res

    def crossover_and_mutate(self, m1, m2, feasible):
        known, _ = self.onepoint_crossover_and_mutation(self.knob_names, m1, m2, feasible)
        known = {k: known[k] for k in self.knob_names}
        res, valid = self.validate(known)
        return res, valid

    def crossover_and_mutate_all(self, m1, m2, feasible):
        keys = list(m1.solved_knob_vals_genotype.keys())
        known, res = self.onepoint_crossover_and_mutation(keys, m1, m2, feasible)
        self.solved_knob_vals_genotype = known
        self.solved_knob_vals_phenotype = known
        score = self.solver.SATScore(known)
        self._valid = score == 0
        return res, self._valid, score

    def satdecoding_crossover_and_mutate(self, m1, m2, feasible):
        keys = list(m1.solved_knob_vals_genotype.keys())
        genotype_dict, _ = self.onepoint_crossover_and_mutation(keys, m1, m2, feasible)
        self.solved_knob_vals_genotype = genotype_dict
        valid, phenotype = self.solver.repair(genotype_dict)
        self._valid = valid
        assert valid
        for idx, key in enumerate(list(self.solver.vals.keys())):
            self.solved_knob_vals_phenotype[key] = phenotype[idx]
        return phenotype, valid

    def SBX_crossover_and_mutation(self, m1, m2, feasible):
        """Simulated binary crossover + polynomial mutation over every model variable, snapped to
        the values seen feasible for that variable; the child may violate constraints, its
        per-constraint violations are returned (knobManager.py:382-423; used by IDEA)."""
        import math
        eta_c, eta_m = 15, 20
        chrom, res = {}, []
        for key in m1.solved_knob_vals_genotype.keys():
            x1, x2 = m1.solved_knob_vals_genotype[key], m2.solved_knob_vals_genotype[key]
            cands = feasible.get(key) or [x1, x2]
            u = random.random()
            sign = float(random.randint(0, 1) * 2 - 1)
            beta = math.pow(2 * u, 1 / eta_c + 1) if u <= 0.5 else math.pow(1 / (2 * (1 - u + 1e-8)), 1 / eta_c + 1)
            x = 0.5 * ((1 + sign * beta) * x1 + (1 - sign * beta) * x2)
            x = min(cands, key=lambda t: abs(t - x))
            if random.random() < 0.1:
                span = max(cands) - min(cands)
                r = random.random()
                delta = math.pow(2 * r, 1 / (eta_m + 1)) - 1 if r < 0.5 else 1 - math.pow(2 * (1 - r), 1 / (eta_m + 1))
                x = min(cands, key=lambda t: abs(t - (x + span * delta)))
            chrom[key] = x
            res.append(x)
        violations, valid = self.solver.MultiSATScore(chrom)
        self.solved_knob_vals_genotype = chrom
        self.solved_knob_vals_phenotype = chrom
        self._valid = valid
        return res, valid, violations

    def constrained_random_walk(self, knob_manager, ratio):
        keys = list(knob_manager.solved_knob_vals_genotype.keys())
        preserve_num = int(ratio * len(keys))
        positions = set(np.random.choice(len(keys), preserve_num, replace=False).tolist())
        known = {key: [knob_manager.solved_knob_vals_genotype[key]]
                 for idx, key in enumerate(keys) if idx in positions}
        valid, res = self.randSample(known)
        return res, valid

    def random_walk(self, knob_manager, feasible):
        knob_name = self.knob_names[random.randint(0, len(self.knob_names) - 1)]
        candidates = feasible[knob_name]
        val = candidates[random.randint(0, len(candidates) - 1)]
        new_knobs = {name: (val if name == knob_name else knob_manager.solved_knob_vals_genotype[name])
                     for name in self.knob_names}
        point = [new_knobs[name] for name in self.knob_names]
        res, valid = self.validate(new_knobs)
        return (res if valid else point), valid

    def valid(self):
        return self._valid
