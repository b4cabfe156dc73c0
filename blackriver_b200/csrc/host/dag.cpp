#include "dag.hpp"

#include <cctype>
#include <cstdlib>
#include <optional>

#include "context.hpp"
#include "tensortype.hpp"

namespace br {

std::ostream& operator<<(std::ostream& os, const Cell& c) {
    if (c.is_string()) os << "S:" << c.as_string();
    else if (c.is_number()) os << "N:" << std::fixed << c.as_number();
    else os << "T: (" << c.as_tensor()->to_string() << " )";
    return os;
}

std::ostream& operator<<(std::ostream& os, const Stack& s) {
    os << "----STACK(" << s.size() << ")----\n";
    size_t i = 0;
    for (auto& c : s.cells()) os << "==>" << i++ << " " << c << "\n";
    os << "----\n";
    return os;
}

// ------------------------------------------------------------------------------------------
// tokenizer
// ------------------------------------------------------------------------------------------
static void tokenize_line(const std::string& line, std::vector<std::string>& out) {
    std::string cur;
    char quote = 0;
    auto flush = [&]() {
        if (!cur.empty()) {
            out.push_back(cur);
            cur.clear();
        }
    };
    for (char ch : line) {
        if (quote) {
            cur.push_back(ch);
            if (ch == quote) {
                out.push_back(cur);
                cur.clear();
                quote = 0;
            }
            continue;
        }
        if (std::isspace((unsigned char)ch) || ch == '(' || ch == ')' || ch == '{' || ch == '}') {
            flush();
        } else if (ch == '[' || ch == ']') {
            flush();
            out.emplace_back(1, ch);
        } else if (ch == '"' || ch == '\'') {
            if (!cur.empty()) br_panic("a string literal must start a token: " + line);
            quote = ch;
            cur.push_back(ch);
        } else if (ch == ';') {
            flush();
            return;
        } else {
            cur.push_back(ch);
        }
    }
    if (quote) br_panic("a string literal must end on its own line: " + line);
    flush();
}

static bool parse_number(const std::string& tok, double& value) {
    bool digit0 = std::isdigit((unsigned char)tok[0]);
    bool neg = tok[0] == '-' && tok.size() >= 2 && std::isdigit((unsigned char)tok[1]);
    if (!digit0 && !neg) return false;
    if (tok.find('.') != std::string::npos || tok.find('e') != std::string::npos) value = std::atof(tok.c_str());
    else value = (double)std::atol(tok.c_str());
    return true;
}

static bool valid_word_name(const std::string& s) {
    static const char* reserved[] = {"true", "ture", "false", "null", "@", "!", "!!", "#", "##"};
    for (auto r : reserved)
        if (s == r) return false;
    if (s.empty() || std::isdigit((unsigned char)s[0])) return false;
    for (char c : s)
        if (!(std::isalnum((unsigned char)c) || c == '_')) return false;
    return true;
}

// ------------------------------------------------------------------------------------------
// compile: text -> items of the main program; %def bodies go to users_
// ------------------------------------------------------------------------------------------
Enviroment::Word Enviroment::compile(const std::string& txt) {
    std::vector<std::string> tokens;
    {
        std::istringstream in(txt);
        std::string line;
        while (std::getline(in, line)) tokenize_line(line, tokens);
    }
    Word main_code;
    std::optional<Word> def_body;
    std::string def_name;
    std::optional<size_t> list_items;

    for (size_t i = 0; i < tokens.size(); i++) {
        const std::string& tok = tokens[i];
        if (tok == "%def") {
            if (def_body) br_panic("%def inside %def");
            if (list_items) br_panic("%def inside a [ ] list");
            if (++i >= tokens.size()) br_panic("%def without a name");
            def_name = tokens[i];
            if (!valid_word_name(def_name) || has_word(def_name)) br_panic("bad or duplicate word name: " + def_name);
            def_body = Word();
            continue;
        }
        if (tok == "%end") {
            if (list_items) br_panic("%end inside a [ ] list");
            if (!def_body) br_panic("%end without %def");
            users_[def_name] = *def_body;
            def_body.reset();
            continue;
        }
        Word& target = def_body ? *def_body : main_code;
        if (tok == "[") {
            if (list_items) br_panic("nested [ ] list");
            list_items = 0;
            continue;
        }
        if (tok == "]") {
            if (!list_items) br_panic("] without [");
            target.push_back({INumber, "", (double)*list_items});
            list_items.reset();
            continue;
        }
        Item it;
        double num;
        if (tok == "ture" || tok == "true") it = {INumber, "", 1.0};
        else if (tok == "false") it = {INumber, "", 0.0};
        else if (tok == "null") it = {IString, "", 0};
        else if (tok == "@" || tok == "!" || tok == "!!" || tok == "#" || tok == "##") it = {IBuiltin, tok, 0};
        else if (tok[0] == '"' || tok[0] == '\'') {
            br_assert(tok.size() >= 2 && tok.front() == tok.back(), "malformed string literal");
            it = {IString, tok.substr(1, tok.size() - 2), 0};
        } else if (tok[0] == '$') it = {IString, tok, 0};
        else if (parse_number(tok, num)) it = {INumber, "", num};
        else if (natives_.count(tok)) it = {INative, tok, 0};
        else if (users_.count(tok)) it = {IUser, tok, 0};
        else br_panic("unknown symbol (not a string, number, builtin, user or native word): " + tok);
        if (list_items) *list_items += 1;
        target.push_back(std::move(it));
    }
    if (list_items) br_panic("[ without ]");
    if (def_body) br_panic("%def without %end");
    return main_code;
}

// ------------------------------------------------------------------------------------------
// link: inline user words, instantiate natives
// ------------------------------------------------------------------------------------------
void Enviroment::link(DaG& dag, const Word& w, int depth) {
    br_assert(depth < 256, "user words nest too deeply");
    for (const Item& it : w) {
        DaG::Op op;
        switch (it.kind) {
            case INumber:
                op.kind = DaG::PushNumber;
                op.num = it.num;
                dag.code_.push_back(op);
                break;
            case IString:
                op.kind = DaG::PushString;
                op.str = it.text;
                dag.code_.push_back(op);
                break;
            case IBuiltin:
                if (it.text == "@") op.kind = DaG::Get;
                else if (it.text == "!") op.kind = DaG::Set;
                else if (it.text == "!!") op.kind = DaG::Drop;
                else if (it.text == "#") op.kind = DaG::ChangeHash;
                else op.kind = DaG::CurrentHash;
                dag.code_.push_back(op);
                break;
            case INative: {
                auto f = natives_.find(it.text);
                br_assert(f != natives_.end(), "native word vanished: " + it.text);
                op.kind = DaG::Native;
                op.idx = dag.natives_.size();
                op.str = it.text;
                dag.natives_.push_back(f->second(*this));
                dag.code_.push_back(op);
                break;
            }
            case IUser: {
                auto f = users_.find(it.text);
                br_assert(f != users_.end(), "user word vanished: " + it.text);
                link(dag, f->second, depth + 1);
                break;
            }
        }
    }
}

Enviroment::Enviroment(int hash_num) {
    br_assert(hash_num >= 1, "at least one hash table");
    hashes_.resize((size_t)hash_num);
    load_base_words();
}

void Enviroment::insert_native_word(const std::string& name, NativeCreator* fn) {
    if (natives_.count(name)) br_panic("native word registered twice: " + name);
    natives_[name] = fn;
}

DaG* Enviroment::build(const std::string& txt) {
    auto dag = std::make_unique<DaG>(this);
    Word code = compile(txt);
    link(*dag, code, 0);
    return dag.release();
}

void Enviroment::run(DaG* dag) {
    br_assert(dag && dag->env_ == this, "program was built by another environment");
    for (const DaG::Op& op : dag->code_) {
        switch (op.kind) {
            case DaG::PushNumber: stack_.push_number(op.num); break;
            case DaG::PushString: stack_.push_string(op.str); break;
            case DaG::Get: stack_.push(Hash::Item2Cell(hash().find(stack_.pop_string()))); break;
            case DaG::Set: {
                std::string name = stack_.pop_string();
                Cell value = stack_.pop();
                hash().set(name, Hash::Cell2Item(value));
                break;
            }
            case DaG::Drop: hash().drop(stack_.pop_string()); break;
            case DaG::ChangeHash: change((size_t)stack_.pop_number()); break;
            case DaG::CurrentHash: stack_.push_number((double)target_); break;
            case DaG::Native:
                if (trace_) trace_(op.str.c_str(), true);
                dag->natives_[op.idx]->run(stack_);
                if (trace_) trace_(op.str.c_str(), false);
                break;
        }
    }
}

void Enviroment::execute(const std::string& txt) {
    DaG dag(this);
    Word code = compile(txt);
    link(dag, code, 0);
    run(&dag);
}

// ------------------------------------------------------------------------------------------
// base words (blackriver/dag.cpp:538-556)
// ------------------------------------------------------------------------------------------
namespace base {
#define BR_STACK_WORD(NAME, BODY)               \
    struct NAME : public NativeWord {           \
        void run(Stack& stack) override { BODY; } \
        NWORD_CREATOR_DEFINE_LR(NAME)           \
    };
BR_STACK_WORD(Drop, stack.drop())
BR_STACK_WORD(Dup, stack.dup())
BR_STACK_WORD(Dup2, stack.dup2())
BR_STACK_WORD(Swap, stack.swap())
BR_STACK_WORD(Rot, stack.rot())
BR_STACK_WORD(Show, std::cout << stack << std::endl)
BR_STACK_WORD(Exit, std::exit(0))
#define BR_ARITH_WORD(NAME, EXPR)                 \
    struct NAME : public NativeWord {             \
        void run(Stack& stack) override {         \
            double a = stack.pop_number();        \
            double b = stack.pop_number();        \
            stack.push_number(EXPR);              \
        }                                         \
        NWORD_CREATOR_DEFINE_LR(NAME)             \
    };
BR_ARITH_WORD(Add, b + a)
BR_ARITH_WORD(Sub, b - a)
BR_ARITH_WORD(Mul, b* a)
BR_ARITH_WORD(Div, b / a)
BR_ARITH_WORD(IntDiv, (double)(int)(b / a))
struct Concat : public NativeWord {
    void run(Stack& stack) override {
        std::string a = stack.pop_string();
        std::string b = stack.pop_string();
        stack.push_string(b + a);
    }
    NWORD_CREATOR_DEFINE_LR(Concat)
};
struct Echo : public NativeWord {
    void run(Stack& stack) override {
        std::string msg = stack.pop_string();
        std::cout << CollectiveContext::mpi_rank << ":" << CollectiveContext::now() << "\t" << msg << std::endl;
    }
    NWORD_CREATOR_DEFINE_LR(Echo)
};
}  // namespace base

void Enviroment::load_base_words() {
    insert_native_word("drop", base::Drop::creator);
    insert_native_word("dup", base::Dup::creator);
    insert_native_word("dup2", base::Dup2::creator);
    insert_native_word("swap", base::Swap::creator);
    insert_native_word("rot", base::Rot::creator);
    insert_native_word("?", base::Show::creator);
    insert_native_word("^", base::Exit::creator);
    insert_native_word("+", base::Add::creator);
    insert_native_word("-", base::Sub::creator);
    insert_native_word("*", base::Mul::creator);
    insert_native_word("/", base::Div::creator);
    insert_native_word("//", base::IntDiv::creator);
    insert_native_word("|", base::Concat::creator);
    insert_native_word("echo", base::Echo::creator);
}

}  // namespace br
