from .ga_tuner import CGATuner, GATuner, RCGATuner, SDGATuner
from .random_tuner import CRandTuner
from .sa_tuner import ConstrainedRandomWalkerSATuner, RandomWalkSATuner, SATuner
from .tuner import Tuner
