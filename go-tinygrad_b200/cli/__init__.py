"""Command-line front end (``bin/llmgen``)."""
