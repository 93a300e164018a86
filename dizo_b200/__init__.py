"""B200-native zeroth-order fine-tuning framework (MeZO estimator, DiZO projection, OPT models)."""
__version__ = "0.1.0"
