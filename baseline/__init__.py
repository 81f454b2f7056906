"""Helpers around the unmodified reference install (``baseline/_ref``); not part of the product."""
