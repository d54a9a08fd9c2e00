import random


def generate(words=2, separator="_"):
    return separator.join(random.choice(["amber", "brisk", "calm", "deft"]) for _ in range(words))
