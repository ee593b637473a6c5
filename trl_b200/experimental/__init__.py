"""Incubating trainers and utilities (counterpart of trl/experimental/__init__.py).  Anything here may change without
deprecation.  Set TRL_EXPERIMENTAL_SILENCE=1 to silence the import notice."""
import os
import warnings


class TRLExperimentalWarning(UserWarning):
    pass


if not os.environ.get("TRL_EXPERIMENTAL_SILENCE"):
    warnings.warn("You are importing from 'trl_b200.experimental'. APIs here are unstable and may change or be removed "
                  "without notice. Silence this warning by setting environment variable TRL_EXPERIMENTAL_SILENCE=1.",
                  TRLExperimentalWarning, stacklevel=2)
