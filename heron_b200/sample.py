"""A candidate point of a task's knob space (sample.py of the reference).

``point`` is the full solved variable vector (also the cost model's feature vector,
model/xgboost_cost_model.py:99-104 of the reference); ``stmt_code`` is its string identity used for
de-duplication (utils.py:306-311); ``perf`` = ln(1/seconds) once measured, 0 if the candidate
failed (runner/runner.py:13-18).
"""
import copy

from .utils import Code, DeCode


class Sample:
    def __init__(self, task):
        self.valid = False
        self.perf = 0.0
        self.task = task
        self.knob_manager = copy.deepcopy(task.knob_manager)
        self.predict = 0
        self.prob = 0
        self.violation = None
        self.violations = None
        self.ranks = []
        self.point = None
        self.stmt_code = None

    def getTask(self):
        return self.task

    def set_point(self, point, valid):
        self.point = list(point)
        self.valid = bool(valid)
        self.stmt_code = Code(self.point)
        return self

    def fromCode(self, code):
        point = DeCode(code)
        self.point = point
        for idx, key in enumerate(list(self.knob_manager.solver.vals.keys())):
            self.knob_manager.solved_knob_vals_genotype[key] = point[idx]
            self.knob_manager.solved_knob_vals_phenotype[key] = point[idx]
        self.stmt_code = code

    def lower(self):
        """Text of the instantiated kernel (the reference lowers to TIR here)."""
        return self.task.getStmt(self.knob_manager)
