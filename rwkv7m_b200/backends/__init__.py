"""Independent re-statements of the model used as parity oracles."""
