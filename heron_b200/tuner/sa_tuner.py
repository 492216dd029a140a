"""Simulated-annealing tuners (tuner/sa_tuner.py of the reference): walk every member of the
population one step and keep the step when the cost model prefers it."""
import math

import numpy as np

from .tuner import Tuner


class SATuner(Tuner):
    def __init__(self, config):
        super().__init__(config)
        self.t = self.config.temperature
        total_iters = math.ceil(self.config.max_trials / self.config.measure_time_per_round) * self.config.iter_walks
        self.cool = self.t / (total_iters + 1)

    def optimize(self, env, population, stat, s_time):
        all_samples = [] + population
        for _ in range(self.config.iter_walks):
            if hasattr(self.cost_model, "bst") and self.cost_model.bst is None:
                break
            stepped = self.walk(population, env)
            population = self.accept(population, stepped, self.t)
            all_samples += population
            self.t -= self.cool
            self.recordStat(all_samples, env, s_time, stat)
        return population, all_samples

    def accept(self, pop, pop1, temp):
        # the reference computes a Metropolis probability and then overrides it with a plain
        # "better than before" test (sa_tuner.py:41-45); the effective rule is the latter
        return [b if b.predict > a.predict else a for a, b in zip(pop, pop1)]


class ConstrainedRandomWalkerSATuner(SATuner):
    def walk(self, pop, env):
        return self.constrained_random_walk(env.task, pop, 1, ratio=0.3)


class RandomWalkSATuner(SATuner):
    def walk(self, pop, env):
        return self.random_walk(env.task, pop, 1, self.feasible)
