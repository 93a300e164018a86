"""Prompt templates: how a task sample becomes text, with and without its answer.

Each template is described by three pieces - ``body`` (the prompt without an answer), an
``answer`` formatter (how a candidate is appended) and the same pair for surface-form
calibration (SFC, where the input is left out) - and compiled into a class exposing the four
methods the rest of the code calls: ``encode``, ``verbalize``, ``encode_sfc``,
``verbalize_sfc``.  The produced strings are those of the reference's templates
(large_models/templates.py:1-400), which follow PromptSource / MeZO conventions.
"""
from __future__ import annotations

from typing import Callable


class Template:
    """Base behaviour: the candidate itself is the verbalisation; SFC input is ``<mask>``."""
    verbalizer: dict | None = None

    def encode(self, sample) -> str:
        raise NotImplementedError

    def verbalize(self, sample, candidate) -> str:
        return candidate

    def encode_sfc(self, sample) -> str:
        return "<mask>"

    def verbalize_sfc(self, sample, candidate) -> str:
        return candidate


def _word(template, candidate):
    return template.verbalizer[candidate] if template.verbalizer else candidate


def _make(name: str, body: Callable, sep: str = "", verbalizer: dict | None = None,
          sfc_body: Callable | None = None, sfc_sep: str | None = None, doc: str = "") -> type:
    """Compile a template class: verbalize = body + sep + word, SFC likewise."""
    sfc_body = sfc_body or (lambda s: "")
    sfc_sep = sep if sfc_sep is None else sfc_sep

    def encode(self, sample):
        return body(sample)

    def verbalize(self, sample, candidate):
        return body(sample) + sep + _word(self, candidate)

    def encode_sfc(self, sample):
        return sfc_body(sample)

    def verbalize_sfc(self, sample, candidate):
        return sfc_body(sample) + sfc_sep + _word(self, candidate)

    return type(name, (Template,), dict(verbalizer=verbalizer, encode=encode, verbalize=verbalize,
                                        encode_sfc=encode_sfc, verbalize_sfc=verbalize_sfc,
                                        __doc__=doc))


# ------------------------------------------------------------------------------- SST-2
SST2Template = _make(
    "SST2Template", lambda s: f"{s.data['sentence'].strip()} It was", sep=" ",
    verbalizer={0: "terrible", 1: "great"}, sfc_body=lambda s: " It was", sfc_sep=" ",
    doc="Sentiment: '<sentence> It was terrible|great'.")


# ------------------------------------------------------------------------------- COPA
class CopaTemplate(Template):
    """'<premise> so|because <choice>' with the choice's first word lower-cased."""
    capitalization: str = "correct"
    effect_conj: str = " so "
    cause_conj: str = " because "

    def get_conjucture(self, sample):
        q = sample.data["question"]
        if q == "effect":
            return self.effect_conj
        if q == "cause":
            return self.cause_conj
        raise NotImplementedError(q)

    def get_prompt(self, sample):
        premise = sample.data["premise"].rstrip()
        if premise.endswith("."):
            premise = premise[:-1]
        prompt = premise + self.get_conjucture(sample)
        if self.capitalization == "upper":
            return prompt.upper()
        if self.capitalization == "lower":
            return prompt.lower()
        return prompt

    def capitalize(self, c):
        mode = self.capitalization
        if mode == "correct":
            words = c.split(" ")
            if words[0] != "I":
                words[0] = words[0].lower()
            return " ".join(words)
        if mode == "bug":
            return c
        if mode == "upper":
            return c.upper()
        if mode == "lower":
            return c.lower()
        raise NotImplementedError(mode)

    def encode(self, sample):
        return self.get_prompt(sample)

    def verbalize(self, sample, candidate):
        return self.get_prompt(sample) + self.capitalize(candidate)

    def encode_sfc(self, sample):
        return self.get_conjucture(sample).strip()

    def verbalize_sfc(self, sample, candidate):
        return self.get_conjucture(sample).strip() + " " + self.capitalize(candidate)


# ------------------------------------------------------------------------------- BoolQ
def _boolq_body(tail: str):
    def body(s):
        q = s.data["question"]
        if not q.endswith("?"):
            q = q + "?"
        q = q[0].upper() + q[1:]
        return f"{s.data['passage']} {q}{tail}"
    return body


BoolQTemplate = _make("BoolQTemplate", _boolq_body(""), sep=" ", sfc_sep="")
BoolQTemplateV2 = _make("BoolQTemplateV2", _boolq_body("\\n\\n"), sfc_sep="")   # literal backslash-n
BoolQTemplateV3 = _make("BoolQTemplateV3", _boolq_body("\n"), sfc_sep="")

# ------------------------------------------------------------------------------- MultiRC / CB / MNLI / WIC / WSC / RTE
MultiRCTemplate = _make(
    "MultiRCTemplate",
    lambda s: (f"{s.data['paragraph']}\nQuestion: {s.data['question']}\nI found this answer "
               f"\"{s.data['answer']}\". Is that correct? Yes or No?\n"),
    verbalizer={0: "No", 1: "Yes"})


def _nli_body(s):
    return (f"Suppose {s.data['premise']} Can we infer that \"{s.data['hypothesis']}\"? "
            f"Yes, No, or Maybe?\n")


CBTemplate = _make("CBTemplate", _nli_body, verbalizer={0: "Yes", 1: "No", 2: "Maybe"})
MNLITemplate = _make("MNLITemplate", _nli_body, verbalizer={0: "Yes", 1: "No", 2: "Maybe"})

WICTemplate = _make(
    "WICTemplate",
    lambda s: (f"Does the word \"{s.data['word']}\" have the same meaning in these two sentences? "
               f"Yes, No?\n{s.data['sentence1']}\n{s.data['sentence2']}\n"),
    verbalizer={0: "No", 1: "Yes"})

WSCTemplate = _make(
    "WSCTemplate",
    lambda s: (f"{s.data['text']}\nIn the previous sentence, does the pronoun "
               f"\"{s.data['span2_text'].lower()}\" refer to {s.data['span1_text']}? Yes or No?\n"),
    verbalizer={0: "No", 1: "Yes"})

RTETemplate = _make(
    "RTETemplate",
    lambda s: (f"{s.data['premise']}\nDoes this mean that \"{s.data['hypothesis']}\" is true? "
               f"Yes or No?\n"),
    verbalizer={0: "Yes", 1: "No"})

# ------------------------------------------------------------------------------- ReCoRD
ReCoRDTemplate = _make(
    "ReCoRDTemplate",
    lambda s: (f"{s.data['passage']}\n{s.data['query']}\nQuestion: what is the \"@placeholder\"\n"
               f"Answer:"),
    sep=" ", sfc_body=lambda s: "Answer:", sfc_sep=" ")


class ReCoRDTemplateGPT3(Template):
    """GPT-3 style cloze: highlights become bullets and the query, with the candidate filled
    in for the placeholder, is the last bullet."""

    @staticmethod
    def _passage(sample):
        return sample.data["passage"].replace("@highlight\n", "- ")

    @staticmethod
    def _query(sample, candidate):
        c = candidate[0] if isinstance(candidate, list) else candidate
        return sample.data["query"].replace("@placeholder", c)

    def encode(self, sample):
        return f"{self._passage(sample)}\n-"

    def verbalize(self, sample, candidate):
        return f"{self._passage(sample)}\n- {self._query(sample, candidate)}"

    def encode_sfc(self, sample):
        return "-"

    def verbalize_sfc(self, sample, candidate):
        return f"- {self._query(sample, candidate)}"


# ------------------------------------------------------------------------------- generation tasks
class _GoldAnswerTemplate(Template):
    """Generation tasks: ``verbalize`` appends the first gold answer and a newline; SFC is
    not defined for them."""

    def _body(self, sample) -> str:
        raise NotImplementedError

    def encode(self, sample):
        return self._body(sample)

    def verbalize(self, sample, candidate):
        return f"{self._body(sample)} {sample.data['answers'][0]}\n"

    def encode_sfc(self, sample):
        raise NotImplementedError

    def verbalize_sfc(self, sample, candidate):
        raise NotImplementedError


class SQuADv2Template(_GoldAnswerTemplate):
    def _body(self, sample):
        d = sample.data
        return f"Title: {d['title']}\nContext: {d['context']}\nQuestion: {d['question'].strip()}\nAnswer:"


class DROPTemplate(_GoldAnswerTemplate):
    def _body(self, sample):
        d = sample.data
        return f"Passage: {d['context']}\nQuestion: {d['question'].strip()}\nAnswer:"
