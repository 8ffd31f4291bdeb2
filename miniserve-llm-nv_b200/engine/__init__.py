"""The engine: step function, scheduler, request state and the entry points above them."""
