"""Genetic tuners (tuner/ga_tuner.py of the reference).

``CGATuner`` is the reference's headline method: constrained crossover + mutation.  Each
generation picks a random 20 % of *all* model variables as key variables; a child must take each
key variable's value from one of its two parents, except one (the mutation), and the constraint
solver completes the rest of the point, so every child is feasible by construction
(ga_tuner.py:68-92, knobManager.py:326-339).
"""
import random
import time

from ..sample import Sample
from .tuner import Tuner, _fan_out


class GATuner(Tuner):
    def optimize(self, env, population, stat, s_time):
        all_pop = [] + population
        for _ in range(self.config.iter_walks):
            if hasattr(self.cost_model, "bst") and self.cost_model.bst is None:
                break  # nothing to optimise against before the first measurements
            self.inferKeyVariables(env, population)
            population = self.RankPop(population)
            population = self.Selection(population, self.config.select_num)
            population = self.crossoverAndMutate(population, env.task)
            all_pop += population
            self.recordStat(all_pop, env, s_time, stat)
            population = population + sorted(all_pop, key=lambda x: x.predict)[-20:]
        self.removeInvalid(all_pop)
        return population, all_pop

    def inferKeyVariables(self, env, pop):
        return

    def RankPop(self, pop):
        return pop

    def Selection(self, pop, num):
        return self.RouletteWheelSelection(pop, num)

    def removeInvalid(self, all_pop):
        for sample in all_pop:
            if not sample.valid:
                sample.predict = 0.0

    def _breed(self, kind, samples, task, args):
        if self.config.parallel:
            workers = max(1, self.config.parallel_num)
            load = (self.config.pop_num + workers - 1) // workers
            res = _fan_out(crossoverAndMutateSequential, [(kind, load, samples, task, args)] * workers, 100)
        else:
            res = crossoverAndMutateSequential(kind, self.config.pop_num, samples, task, args)
        return self._score(res)

    def crossoverAndMutate(self, samples, task):
        return self._breed("Unconstrained", samples, task, self.feasible)


class CGATuner(GATuner):
    def check_feasible_exits(self, env, num=1e3):
        return  # constrained operators never leave the feasible set: no value table needed

    def inferKeyVariables(self, env, pop):
        names = list(env.task.knob_manager.solver.vals.keys())
        random.shuffle(names)
        self.key_variables = names[: int(self.config.crossover_key_ratio * len(names))]

    def crossoverAndMutate(self, samples, task):
        keys = getattr(self, "key_variables", None)
        if keys is None:
            names = list(task.knob_manager.solver.vals.keys())
            random.shuffle(names)
            keys = names[: int(self.config.crossover_key_ratio * len(names))]
        return self._breed("Constrained", samples, task, keys)


class RCGATuner(CGATuner):
    """CGA with a fresh random key set for every breeding call."""

    def inferKeyVariables(self, env, pop):
        self.key_variables = None


class SDGATuner(GATuner):
    """Unconstrained crossover repaired into the feasible set by the solver (SAT decoding)."""

    def crossoverAndMutate(self, samples, task):
        return self._breed("SATDecoding", samples, task, self.feasible)


class SRGATuner(GATuner):
    """GA over all variables with stochastic ranking between fitness and constraint violation
    (ga_tuner.py:113-152 of the reference)."""

    def Selection(self, pop, num):
        return self.RankSelection(pop, num)

    def RankPop(self, pop):
        sweeps, pf = 10, 0.45
        order = list(pop)
        for _ in range(sweeps):
            swapped = False
            for j in range(len(order) - 1):
                a, b = order[j], order[j + 1]
                va, vb = a.violation or 0, b.violation or 0
                by_fitness = (va == 0 and vb == 0) or random.random() < pf
                if (by_fitness and a.predict < b.predict) or (not by_fitness and va > vb):
                    order[j], order[j + 1] = b, a
                    swapped = True
            if not swapped:
                break
        return order

    def crossoverAndMutate(self, samples, task):
        res = self._breed("UnconstrainedAll", samples, task, self.feasible)
        for s in res:  # infeasible children keep a (penalised) predicted fitness for the ranking
            if not s.valid and s.point is not None:
                s.predict = float(self.predict([s])[0]) if self.cost_model is not None else 0.0
        return res


def crossoverAndMutateSequential(kind, num, samples, task, args):
    res = []
    for _ in range(num):
        m1 = samples[random.randint(0, len(samples) - 1)].knob_manager
        m2 = samples[random.randint(0, len(samples) - 1)].knob_manager
        child = Sample(task)
        km = child.knob_manager
        violation = None
        if kind == "Constrained":
            point, valid = km.constrained_crossover_and_mutate(m1, m2, args)
        elif kind == "Unconstrained":
            point, valid = km.crossover_and_mutate(m1, m2, args)
        elif kind == "UnconstrainedAll":
            point, valid, violation = km.crossover_and_mutate_all(m1, m2, args)
        elif kind == "SATDecoding":
            point, valid = km.satdecoding_crossover_and_mutate(m1, m2, args)
        elif kind == "SBX":
            point, valid, child.violations = km.SBX_crossover_and_mutation(m1, m2, args)
        else:
            raise ValueError(kind)
        child.violation = violation
        res.append(child.set_point(point, valid))
    return res
