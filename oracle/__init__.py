"""CPU oracle of the attention path.  Test infrastructure only: nothing under
``nitrix_b200`` imports this package (see ``oracle/sdpa_oracle.py``)."""
