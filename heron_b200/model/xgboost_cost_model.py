"""Cost model behind the reference's ``XGBoostCostModel`` interface
(model/xgboost_cost_model.py:14-104): ``train(perf_buffer)`` fits a gradient-boosted regressor on
(solved variable vector -> normalised fitness), ``predict(samples)`` scores candidates, and an
untrained model predicts 1 for everything so that the first round is a random search.

xgboost is not installed here; scikit-learn's ``GradientBoostingRegressor`` stands in with the
reference's tree depth and learning rate, and with early stopping on the training curve in place
of the reference's recall@N callback.  ``bst`` keeps its meaning (None until trained) and offers
``get_score()`` (feature weights keyed ``f<i>``) because the CGA tuner ranks key variables
through it (utils.py:314-328 of the reference).
"""
import numpy as np


class _Booster:
    def __init__(self, model):
        self.model = model

    def predict(self, x):
        return self.model.predict(x)

    def get_score(self, importance_type="weight"):
        imp = self.model.feature_importances_
        return {"f%d" % i: float(v) for i, v in enumerate(imp) if v > 0}


class XGBoostCostModel:
    def __init__(self, task, config, num_threads=None, log_interval=25):
        self.task = task
        self.target = task.target
        self.loss_type = getattr(config, "loss_type", "reg")
        if self.loss_type not in ("reg", "rank"):
            raise RuntimeError("Invalid loss type: " + self.loss_type)
        self.num_threads = num_threads
        self.log_interval = log_interval
        self.params = dict(max_depth=7 if self.loss_type == "reg" else 3, learning_rate=0.3,
                           n_estimators=300, subsample=1.0, min_samples_leaf=1)
        self.bst = None
        self._sample_size = 0

    def train(self, perf_buffer):
        self.fit(np.array(perf_buffer.data_x), np.array(perf_buffer.data_y))

    def fit(self, x_train, y_train, plan_size=30):
        from sklearn.ensemble import GradientBoostingRegressor
        if len(x_train) < 2:
            return
        y = y_train / (max(y_train) + 1e-8)
        index = np.random.permutation(len(x_train))
        if len(x_train) >= 40:
            model = GradientBoostingRegressor(n_iter_no_change=20, validation_fraction=0.1, tol=1e-6, **self.params)
        else:
            model = GradientBoostingRegressor(**dict(self.params, n_estimators=100))
        model.fit(np.asarray(x_train, dtype=np.float64)[index], y[index])
        self._sample_size = len(x_train)
        self.bst = _Booster(model)

    def predict(self, samples, output_margin=False):
        if self.bst is None:
            return np.ones(len(samples))
        if len(samples) == 0:
            return np.zeros(0)
        feas = np.array([s.point for s in samples], dtype=np.float64)
        return self.bst.predict(feas)
