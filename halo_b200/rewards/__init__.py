"""Reward terms, graders and the composer that turns an episode into one scalar."""
