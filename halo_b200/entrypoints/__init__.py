"""Script lifecycle: parse -> initialise -> build model / data / trainer -> train -> tear down."""
