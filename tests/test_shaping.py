"""Arabic contextual shaping and the visual reordering of mixed-direction lines (``imaging/shaping.py``)."""
import unicodedata

from idrak_b200.imaging import base_direction, layout_line, shape_arabic, visual_order


def _names(s):
    return [unicodedata.name(c) for c in s]


def test_contextual_forms_of_a_joined_word():
    # kaf-teh-alef-beh: kaf initial, teh medial, alef final (and it does not join onward), beh isolated
    got = _names(shape_arabic("كتاب"))
    assert got == ["ARABIC LETTER KAF INITIAL FORM", "ARABIC LETTER TEH MEDIAL FORM",
                   "ARABIC LETTER ALEF FINAL FORM", "ARABIC LETTER BEH ISOLATED FORM"]


def test_lam_alef_ligature_and_marks_are_transparent():
    # seen-lam-alef-meem: the lam and alef fuse into the final-form ligature; meem stands alone after it
    got = _names(shape_arabic("سلام"))
    assert got == ["ARABIC LETTER SEEN INITIAL FORM", "ARABIC LIGATURE LAM WITH ALEF FINAL FORM",
                   "ARABIC LETTER MEEM ISOLATED FORM"]
    assert _names(shape_arabic("لا")) == ["ARABIC LIGATURE LAM WITH ALEF ISOLATED FORM"]
    # a fatha between beh and teh does not break the join
    got = shape_arabic("بَت")
    assert _names(got)[0] == "ARABIC LETTER BEH INITIAL FORM" and _names(got)[2] == "ARABIC LETTER TEH FINAL FORM"
    assert got[1] == "َ"


def test_non_arabic_text_is_untouched_and_single_letters_are_isolated():
    assert shape_arabic("hello, 123") == "hello, 123"
    assert _names(shape_arabic("ب ب")) == ["ARABIC LETTER BEH ISOLATED FORM", "SPACE", "ARABIC LETTER BEH ISOLATED FORM"]


def test_visual_order_of_mixed_lines():
    assert base_direction("abc א") == "L" and base_direction("א abc") == "R" and base_direction("12 !") == "L"
    # a right-to-left word inside a left-to-right line is reversed; the number after it stays in reading order and
    # belongs to the right-to-left run (so it is drawn to the word's left)
    assert visual_order("abc אבג 123 def") == "abc 123 גבא def"
    # a right-to-left line: runs laid out from the right, brackets mirrored inside the reversed run
    assert visual_order("אב (12) ok") == "ok (12) בא"
    assert visual_order("plain") == "plain"


def test_layout_line_shapes_then_reorders():
    out = layout_line("سلام ok")
    assert out.startswith("ok ") and _names(out[3:]) == ["ARABIC LETTER MEEM ISOLATED FORM",
                                                        "ARABIC LIGATURE LAM WITH ALEF FINAL FORM",
                                                        "ARABIC LETTER SEEN INITIAL FORM"]
