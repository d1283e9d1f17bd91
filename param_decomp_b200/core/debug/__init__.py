"""Debugging tools of the engine: launch / collective census, memory ledger, deviceless fit check."""
