"""Python face of the native executor: the op records a model's parts emit
(records.py) and the program that runs them (program.py)."""
