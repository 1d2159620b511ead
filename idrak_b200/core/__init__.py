"""Core API shape over PyTorch: autograd helpers, scopes, mixed precision, activation memory."""
