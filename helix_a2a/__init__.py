"""Drop-in name for users of the reference: ``import helix_a2a`` gives the B200 library.

Same surface as the reference package (``helix_a2a/__init__.py:23-121``):
``workspace_size``, ``allocate_workspace``, ``init_workspace``, ``alltoall``, ``__version__``.
"""
from helix_a2a_b200 import *  # noqa: F401,F403
from helix_a2a_b200 import __all__, __version__  # noqa: F401
