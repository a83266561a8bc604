"""CPU oracle (test infrastructure): numpy restatement in bqq_oracle.py, C restatement in
bqq_oracle.c (loaded through c_oracle.py)."""
