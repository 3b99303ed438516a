"""Mixture-of-experts operators on the B200 weight image."""
