"""Namespace package: callaghandev.ml_b200 is the B200 training back end for CallaghanDev.ML."""
