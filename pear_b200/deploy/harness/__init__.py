"""Agent harness: a session service and an upstream proxy between an agent CLI and the model server."""
