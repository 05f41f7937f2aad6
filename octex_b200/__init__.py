"""octex_b200: the batched search path of hpdic/octex, written for NVIDIA B200 (sm_100a).

``load`` / ``attach`` place an index on the GPU of this process; ``Index.search`` answers a batch of
queries; ``build`` makes an index directory on the GPU.  ``build_index`` (a torch restatement of
the builder that also runs on a CPU) and ``synth`` (seeded synthetic data) are tooling.
The CUDA library is ``octex_b200/lib/liboctex_b200.so``; without it nothing here computes.
"""
from .index import (Index, attach, build, build_native, cell_codes, exact_neighbors,  # noqa: F401
                    index_params, load, load_params, search_params, stored_vectors)

__version__ = "0.1.0"
__all__ = ["Index", "attach", "build", "build_native", "cell_codes", "exact_neighbors", "index_params", "load",
           "load_params", "search_params", "stored_vectors", "__version__"]
