"""Optional integrations built on the public engine API."""
