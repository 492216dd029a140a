from .knobManager import KnobManager
from .primitives import EQ, LE, LT, NE, ProdTwo, Sum
from .solver import Solver, Variable
