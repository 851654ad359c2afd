"""Browser front end over the session store (rollouts/frontend/server.py:47)."""
