from .measure_methods import (MeasureErrorNo, MeasureResult, measure_handle, perf_from_cost, reduce_costs,
                              time_launches)
from .runner import LocalRunner, Runner, measure_option
