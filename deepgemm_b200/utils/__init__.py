from . import math
from .math import *  # noqa: F401,F403
from . import dist  # noqa: F401
from .dist import init_dist, uneven_all_gather  # noqa: F401
