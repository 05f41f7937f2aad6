"""octex_b200: the batched search path of hpdic/octex, written for NVIDIA B200 (sm_100a).

``load`` / ``attach`` place an index on the GPU of this process; ``Index.search`` answers a batch of
queries.  ``build_index`` and ``synth`` are tooling (index directories and seeded synthetic data).
The CUDA library is ``octex_b200/lib/liboctex_b200.so``; without it nothing here computes.
"""
from .index import (Index, attach, build, cell_codes, load, load_params, search_params,  # noqa: F401
                    stored_vectors)

__version__ = "0.1.0"
__all__ = ["Index", "attach", "build", "cell_codes", "load", "load_params", "search_params",
           "stored_vectors", "__version__"]
