"""Constrained random search (tuner/random_tuner.py of the reference): the baseline the
reference calls CRAND."""
from .tuner import Tuner


class CRandTuner(Tuner):
    def optimize(self, env, pop, stat, s_time):
        samples = [] + pop
        population = pop
        for _ in range(self.config.iter_walks):
            population = self.constrained_random_sample(env, self.config.pop_num)
            samples = samples + population
            self.recordStat(samples, env, s_time, stat)
        population = population + sorted(samples, key=lambda x: -x.predict)[:20]
        return population, samples
