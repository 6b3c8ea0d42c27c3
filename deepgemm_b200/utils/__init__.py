from . import math
from .math import *  # noqa: F401,F403
