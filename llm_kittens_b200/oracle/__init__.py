"""Plain-PyTorch reference implementations used as numerical oracle and library baseline."""
