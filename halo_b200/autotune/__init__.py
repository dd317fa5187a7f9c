"""The SQLite kernel autotuner of the matmul path, re-keyed to B200.

File format and semantics follow the reference's src/autotune (schema v1 of src/autotune/db.cpp:55-111, the 12-field
profile key of src/autotune/profile_key.cpp:15-31, candidate text of src/autotune/types.cpp:13-66, winner rules of
src/autotune/tuner.cpp:106-163, lookup order of src/autotune/lookup.cpp:72-148), so that a profile database written
here is one HALO's own ProfileLookup can open: same tables, same application id, rows under backend label "cuda".
"""
from .candidate import Candidate  # noqa: F401
from .db import DbError, ProfileDb  # noqa: F401
from .key import OpKey, ProfileKey, b200_profile_key  # noqa: F401
from .cost_model import CostEstimate, CostInputs, CostModel, calibrate_gflops_per_thread  # noqa: F401
from .tuner import CandidateResult, OpTuneResult, TuneOptions, UnsupportedError, plan_candidates, select_kernel, tune  # noqa: F401
