"""CPU oracle package (test infrastructure only; see tb_oracle.h)."""
