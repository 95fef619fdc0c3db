"""CPU execution of the SRU layer stack with the oracle scan.  TEST INFRASTRUCTURE ONLY.

The model is ``ref_model.OracleSRU``, a self-contained restatement of the reference's layer stack that
does not import the shipped package; ``to_oracle`` builds one from any model object that carries the
reference's attribute and ``state_dict`` names.  This is the model-level checker of the GPU tests and
the CPU baseline that the benchmark times.
"""
from .ref_model import OracleSRU, from_state, sru_kwargs_of, to_oracle  # noqa: F401
