"""Text preprocessing (keras/preprocessing/text.py): a word-index tokenizer."""
import re
from collections import Counter

_FILTERS = '!"#$%&()*+,-./:;<=>?@[\\]^_`{|}~\t\n'


def text_to_word_sequence(text, filters=_FILTERS, lower=True, split=" "):
    if lower:
        text = text.lower()
    text = re.sub("[" + re.escape(filters) + "]", split, text)
    return [w for w in text.split(split) if w]


class Tokenizer:
    """Words are numbered from 1 by falling frequency (ties: first seen first); with `num_words`, only the num_words - 1 most
    frequent ones are kept by texts_to_sequences; `oov_token` takes index 1 and stands in for the others."""

    def __init__(self, num_words=None, filters=_FILTERS, lower=True, split=" ", oov_token=None):
        self.num_words, self.filters, self.lower, self.split, self.oov_token = num_words, filters, lower, split, oov_token
        self.word_counts = Counter()
        self.word_index = {}
        self.index_word = {}

    def fit_on_texts(self, texts):
        for t in texts:
            self.word_counts.update(text_to_word_sequence(t, self.filters, self.lower, self.split))
        first_seen = {w: i for i, w in enumerate(self.word_counts)}
        words = sorted(self.word_counts, key=lambda w: (-self.word_counts[w], first_seen[w]))
        if self.oov_token is not None:
            words = [self.oov_token] + [w for w in words if w != self.oov_token]
        self.word_index = {w: i + 1 for i, w in enumerate(words)}
        self.index_word = {i: w for w, i in self.word_index.items()}

    def texts_to_sequences(self, texts):
        oov = self.word_index.get(self.oov_token) if self.oov_token is not None else None
        out = []
        for t in texts:
            seq = []
            for w in text_to_word_sequence(t, self.filters, self.lower, self.split):
                i = self.word_index.get(w)
                if i is not None and (self.num_words is None or i < self.num_words):
                    seq.append(i)
                elif oov is not None:
                    seq.append(oov)
            out.append(seq)
        return out
