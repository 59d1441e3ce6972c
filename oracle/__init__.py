"""CPU oracle (test infrastructure only; see reference_math.py)."""
