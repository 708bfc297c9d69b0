"""Station: the model session on a robot (observe, ask the model, read the action, execute), its model clients and a simulated arm."""
