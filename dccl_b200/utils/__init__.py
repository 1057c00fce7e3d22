"""Helpers: reference fold, memory wrappers, rank launcher, .tt reader, clock sampling."""
