"""Drop-in name: ``from dfloat11 import DFloat11Model, compress_model`` as in the reference's
README (README.md:63) and examples.  Everything lives in ``dfloat11_b200``."""
from dfloat11_b200 import *  # noqa: F401,F403
from dfloat11_b200 import DFloat11Model, compress_model  # noqa: F401
