"""Search loop shared by every tuner (tuner/tuner.py:12-385 of the reference).

One round = refresh the population (random feasible points + best measured so far + survivors),
let the subclass improve it against the cost model (``optimize``), pick
``measure_time_per_round`` candidates (60 % greedy, 40 % roulette — ``epsilon_select``),
measure them on the device, retrain the cost model, append a line to ``stat.txt``
(round, sample s, measure s, train s, elapsed s, best perf).
"""
import json
import math
import os
import time

import numpy as np

from ..model import XGBoostCostModel
from ..multi import Job
from ..sample import Sample
from ..utils import Code


class Tuner:
    def __init__(self, config):
        self.config = config
        self.iter_no = 0
        self.cost_model = None
        self.total_sample_time = 0
        self.total_measure_time = 0
        self.feasible = {}

    def buildCostModel(self, task):
        self.cost_model = XGBoostCostModel(task, self.config)

    def setPretrainedModel(self, model):
        self.cost_model = model

    def predict(self, samples):
        if self.cost_model is None:
            return np.ones(len(samples))
        res = self.cost_model.predict(samples)
        if isinstance(res, dict):
            return res[list(res.keys())[0]]
        return res

    # -- the loop ------------------------------------------------------------------------------
    def run(self, env, do_measure=True):
        self.check_feasible_exits(env)
        cfg = self.config
        start_time = time.time()
        total_iters = math.ceil(cfg.max_trials / cfg.measure_time_per_round) + 1
        last_iter_select_num = cfg.max_trials % cfg.measure_time_per_round
        population, stat = [], []
        for iter_no in range(total_iters):
            self.iter_no = iter_no
            select_num = last_iter_select_num if iter_no == total_iters - 1 else cfg.measure_time_per_round
            t0 = time.time()
            initial_population = self.UpdatePopulation(env, population)
            population, all_pop = self.optimize(env, initial_population, stat, start_time)
            t1 = time.time()
            pop = self.epsilon_select(env, all_pop, 0.6, select_num)
            if do_measure and pop:
                self.measure(self.FilterSamples(pop, env), env)
            t2 = time.time()
            if iter_no != total_iters - 1 and self.cost_model is not None and len(env.perf_buffer.data_y) > 0 \
                    and do_measure:
                self.cost_model.train(env.perf_buffer)
            t3 = time.time()
            self._write_stat(env, iter_no, t1 - t0, t2 - t1, t3 - t2, time.time() - start_time)
        return population, stat

    def _write_stat(self, env, iter_no, sample_time, measure_time, train_time, cur_time):
        log_dir = getattr(self.config, "log_dir", None)
        if not log_dir or not os.path.isdir(log_dir):
            return
        best_perf = env.perf_buffer.best_perf or 0
        with open(os.path.join(log_dir, "stat.txt"), "a") as f:
            f.write("%d,%f,%f,%f,%f,%f\n" % (iter_no, sample_time, measure_time, train_time, cur_time, best_perf))

    def optimize(self, env, population, stat, s_time):
        raise NotImplementedError()

    def UpdatePopulation(self, env, population, pretrained=False):
        rand = self.constrained_random_sample(env, self.config.pop_num)
        topk = self.history_topk_samples(env, self.config.history_topk)
        if not pretrained:
            self.repredict(population)  # the cost model has changed since these were scored
        all_pop = population + topk + rand
        return sorted(all_pop, key=lambda x: -x.predict)[: self.config.pop_num]

    def measure(self, samples, env):
        env.evalSamples(samples)

    def check_feasible_exits(self, env, sample_num=1000):
        """Per-variable value sets seen in random feasible samples; the unconstrained GA / SA
        variants mutate within them (tuner/tuner.py:115-144).  Cached in ``feasible.json``."""
        path = self.config.feasible_file_path
        log_dir = getattr(self.config, "log_dir", None)
        if log_dir and os.path.isdir(log_dir) and not os.path.isabs(path):
            path = os.path.join(log_dir, path)
        if os.path.exists(path):
            with open(path, "r") as f:
                self.feasible = json.loads(f.read())
            return
        population = self.constrained_random_sample(env, int(sample_num), timeout=200)
        seen = {}
        for sample in population:
            for name, val in sample.knob_manager.solved_knob_vals_phenotype.items():
                seen.setdefault(name, set()).add(val)
        self.feasible = {k: sorted(v) for k, v in seen.items()}
        if log_dir and os.path.isdir(log_dir):
            with open(path, "w") as f:
                f.write(json.dumps(self.feasible))

    # -- selection -----------------------------------------------------------------------------
    def RouletteWheelSelection(self, samples, num):
        if len(samples) <= num:
            return samples
        predicts = np.array([x.predict for x in samples], dtype=np.float64)
        weights = predicts - predicts.min() + 1e-16
        picked = np.random.choice(len(samples), num, p=weights / weights.sum(), replace=True)
        return [samples[i] for i in picked]

    def RankSelection(self, samples, num):
        if len(samples) <= num:
            return samples
        weights = (len(samples) - np.arange(len(samples))).astype(np.float64)
        picked = np.random.choice(len(samples), num, p=weights / weights.sum(), replace=False)
        return [samples[i] for i in picked]

    def recordStat(self, samples, env, start_time, stat):
        samples = self.FilterSamples(samples, env)
        if not samples:
            return
        perfs = sorted((x.predict for x in samples), reverse=True)
        stat.append([time.time() - start_time, perfs[0], sum(perfs[:5]) / len(perfs[:5])])

    def FilterSamples(self, samples, env):
        codes, ret = set(), []
        for sample in samples:
            code = sample.stmt_code
            if code in codes or code in env.perf_buffer.perfs:
                continue
            codes.add(code)
            ret.append(sample)
        return ret

    def epsilon_select(self, env, all_samples, epsilon, select_num):
        filtered = self.FilterSamples(all_samples, env)
        if not filtered or select_num <= 0:
            return []
        ranked = sorted(filtered, key=lambda x: -x.predict)
        k = int(select_num * epsilon)
        return ranked[:k] + self.RouletteWheelSelection(ranked[k:], select_num - k)

    def greedy_select(self, env, all_samples, select_num):
        filtered = self.FilterSamples(all_samples, env)
        return sorted(filtered, key=lambda x: -x.predict)[:select_num]

    # -- sampling ------------------------------------------------------------------------------
    def _score(self, samples):
        valid = [s for s in samples if s.valid]
        if valid:
            for s, p in zip(valid, self.predict(valid)):
                s.predict = p
        for s in samples:
            if not s.valid:
                s.predict = 0
        return samples

    def constrained_random_sample(self, env, number, timeout=10):
        if self.config.parallel:
            samples = constrained_random_sample_parallel(env.task, number, self.config, timeout)
        else:
            samples = constrained_random_sample_sequential(env.task, number, self.config)
        for s in self._score(samples):
            s.violation = 0
        return samples

    def random_walk(self, task, pop, num_per_sample, feasible):
        return self._score(random_walk_sequential("random_walk", task, pop, num_per_sample, [feasible]))

    def constrained_random_walk(self, task, pop, num_per_sample, ratio=0.3):
        return self._score(random_walk_sequential("constrained_random_walk", task, pop, num_per_sample, [ratio]))

    def history_topk_samples(self, env, k):
        pb = env.perf_buffer
        ranked = sorted(zip(pb.data_y, range(len(pb.samples))), key=lambda t: t[0])[-k:]
        ret = []
        for _, idx in ranked:
            sample = pb.samples[idx]
            sample.violation = 0.0
            ret.append(sample)
        return ret

    def repredict(self, pop):
        for sample in pop:
            if sample.valid:
                sample.predict = self.predict([sample])[0]
                sample.violation = 0.0
            else:
                sample.predict = 0.0


def _new_sample(task, point, valid, violation=None):
    s = Sample(task)
    return s, point, valid, violation


def constrained_random_sample_sequential(task, number, config):
    ret = []
    for _ in range(int(number)):
        sample = Sample(task)
        valid, point = sample.knob_manager.randSample({})
        ret.append(sample.set_point(point, valid))
    return ret


def _fan_out(func, chunks, timeout):
    """Runs ``func(*chunk)`` for every chunk in forked workers (the reference's ``Job``) and
    concatenates the lists they return; a worker that times out contributes nothing."""
    jobs = [Job(func, chunk, timeout) for chunk in chunks]
    for job in jobs:
        job.start(job.attach_info)
    res = []
    for job in jobs:
        ret = job.get()
        if isinstance(ret, list):
            res += ret
    return res


def constrained_random_sample_parallel(task, number, config, timeout):
    workers = max(1, min(config.parallel_num, int(number)))
    work_load = int((number + workers - 1) // workers)
    return _fan_out(constrained_random_sample_sequential, [(task, work_load, config)] * workers, timeout)


def random_walk_sequential(kind, task, pop, num_per_sample, args):
    ret = []
    for sample in pop:
        for _ in range(num_per_sample):
            new_sample = Sample(task)
            km = new_sample.knob_manager
            if kind == "random_walk":
                point, valid = km.random_walk(sample.knob_manager, *args)
            elif kind == "constrained_random_walk":
                point, valid = km.constrained_random_walk(sample.knob_manager, *args)
            else:
                raise ValueError(kind)
            ret.append(new_sample.set_point(point, valid))
    return ret
