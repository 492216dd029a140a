from .ga_tuner import CGATuner, GATuner, RCGATuner, SDGATuner, SRGATuner
from .idea_tuner import IDEATuner
from .random_tuner import CRandTuner
from .sa_tuner import ConstrainedRandomWalkerSATuner, RandomWalkSATuner, SATuner
from .tuner import Tuner
