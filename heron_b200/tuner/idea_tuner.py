"""IDEA: infeasibility-driven evolutionary algorithm (tuner/idea_tuner.py of the reference), one of
the unconstrained baselines the reference compares CGA with.

Children come from simulated binary crossover over all variables and may be infeasible.  The
population keeps a fixed share (20 %) of infeasible members; feasible and infeasible members are
each ordered by non-dominated sorting on two objectives — predicted fitness and a constraint
rank (sum over constraints of the member's rank by violation) — with crowding distance inside a
front.
"""
import numpy as np

from .ga_tuner import GATuner


class IDEATuner(GATuner):
    infeasible_share = 0.2

    def optimize(self, env, pop, stat, s_time):
        n_inf = int(self.infeasible_share * len(pop))
        n_f = len(pop) - n_inf
        all_pop = [] + pop
        for _ in range(self.config.iter_walks):
            if hasattr(self.cost_model, "bst") and self.cost_model.bst is None:
                break
            children = self.crossoverAndMutate(pop, env.task)
            merged = pop + children
            feasible = self.Rank([s for s in merged if s.valid])
            infeasible = self.Rank([s for s in merged if not s.valid])
            pop = feasible[:n_f] + infeasible[:n_inf]
            all_pop += children
            self.recordStat(all_pop, env, s_time, stat)
        self.removeInvalid(all_pop)
        return pop, all_pop

    def UpdatePopulation(self, env, population, pretrained=False):
        topk = self.history_topk_samples(env, self.config.history_topk)
        rand = self.constrained_random_sample(env, self.config.pop_num)
        if not pretrained:
            self.repredict(population)
        half = self.config.pop_num // 2
        return (sorted(population + topk, key=lambda x: -x.predict)[:half]
                + sorted(rand, key=lambda x: -x.predict)[:half])

    def crossoverAndMutate(self, samples, task):
        return self._breed("SBX", samples, task, self.feasible)

    # -- ordering --------------------------------------------------------------------------------
    def constraint_measure(self, pop):
        dim = len(pop[0].knob_manager.solver.primitives)
        for s in pop:
            if s.violations is None:
                s.violations = [0] * dim if s.valid else [1e8] * dim
        ranks = np.zeros((len(pop), dim), dtype=np.int64)
        for i in range(dim):
            col = np.array([s.violations[i] for s in pop], dtype=np.float64)
            _, inverse = np.unique(col, return_inverse=True)  # equal violations share a rank
            ranks[:, i] = inverse
        for s, r in zip(pop, ranks.sum(axis=1)):
            s.rank = int(r)

    def Rank(self, pop):
        """Fronts of the (predicted fitness up, constraint rank up) order the reference uses
        (idea_tuner.py:92-110), crowding distance ascending inside a front."""
        if not pop:
            return []
        self.constraint_measure(pop)
        n = len(pop)
        dominated_by = [set() for _ in range(n)]
        counts = [0] * n
        for i in range(n):
            for j in range(i + 1, n):
                a, b = pop[i], pop[j]
                if a.predict == b.predict and a.rank == b.rank:
                    continue
                if a.predict >= b.predict and a.rank >= b.rank:
                    dominated_by[i].add(j)
                    counts[j] += 1
                elif b.predict >= a.predict and b.rank >= a.rank:
                    dominated_by[j].add(i)
                    counts[i] += 1
        front = [i for i in range(n) if counts[i] == 0]
        ordered = []
        while front:
            members = [pop[i] for i in front]
            self.crowdingDist(members)
            ordered += sorted(members, key=lambda s: s.dist)
            nxt = []
            for i in front:
                for j in dominated_by[i]:
                    counts[j] -= 1
                    if counts[j] == 0:
                        nxt.append(j)
            front = nxt
        return ordered

    def crowdingDist(self, pop):
        for s in pop:
            s.dist = 0.0
        if len(pop) < 3:
            for s in pop:
                s.dist = 1e8
            return
        for key in ("predict", "rank"):
            order = sorted(pop, key=lambda s: getattr(s, key))
            lo, hi = getattr(order[0], key), getattr(order[-1], key)
            if key == "predict":
                order[0].dist = order[-1].dist = 1e8
            for a, mid, b in zip(order, order[1:], order[2:]):
                mid.dist += (getattr(b, key) - getattr(a, key)) / (hi - lo + 1e-8)
