"""A B200-native single-GPU inference engine, built after studying filthyrake/damendaemon.

Everything between a request's token ids and its next token, for one architecture
at a time (GPT-2 today), assembled from registered parts so that another
architecture is a new spec builder and, at most, new part kinds.
"""
__version__ = "0.1.0"
