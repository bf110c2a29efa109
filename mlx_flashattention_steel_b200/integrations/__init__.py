"""Caller integrations (role of mlx_mfa/integrations in the reference)."""
